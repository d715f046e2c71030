* c499 (c499: 32-bit single-error-correcting circuit): 192 gates, 2604 transistors
VDD vdd 0 DC 1.8
VIN0 nd0 0 PULSE(0 1.8 5e-10 20p 20p 1e-09 2e-09)
VIN1 nd1 0 PULSE(0 1.8 1e-09 20p 20p 2e-09 4e-09)
VIN2 nd2 0 PULSE(0 1.8 2e-09 20p 20p 4e-09 8e-09)
VIN3 nd3 0 PULSE(0 1.8 4e-09 20p 20p 8e-09 1.6e-08)
VIN4 nd4 0 PULSE(0 1.8 8e-09 20p 20p 1.6e-08 3.2e-08)
VIN5 nd5 0 PULSE(0 1.8 1.6e-08 20p 20p 3.2e-08 6.4e-08)
VIN6 nd6 0 PULSE(0 1.8 3.2e-08 20p 20p 6.4e-08 1.28e-07)
VIN7 nd7 0 PULSE(0 1.8 6.4e-08 20p 20p 1.28e-07 2.56e-07)
VIN8 nd8 0 PULSE(0 1.8 1.28e-07 20p 20p 2.56e-07 5.12e-07)
VIN9 nd9 0 PULSE(0 1.8 2.56e-07 20p 20p 5.12e-07 1.024e-06)
VIN10 nd10 0 PULSE(0 1.8 5.12e-07 20p 20p 1.024e-06 2.048e-06)
VIN11 nd11 0 PULSE(0 1.8 1.024e-06 20p 20p 2.048e-06 4.096e-06)
VIN12 nd12 0 PULSE(0 1.8 2.048e-06 20p 20p 4.096e-06 8.192e-06)
VIN13 nd13 0 PULSE(0 1.8 4.096e-06 20p 20p 8.192e-06 1.6384e-05)
VIN14 nd14 0 PULSE(0 1.8 8.192e-06 20p 20p 1.6384e-05 3.2768e-05)
VIN15 nd15 0 PULSE(0 1.8 1.6384e-05 20p 20p 3.2768e-05 6.5536e-05)
VIN16 nd16 0 PULSE(0 1.8 3.2768e-05 20p 20p 6.5536e-05 0.000131072)
VIN17 nd17 0 PULSE(0 1.8 6.5536e-05 20p 20p 0.000131072 0.000262144)
VIN18 nd18 0 PULSE(0 1.8 0.000131072 20p 20p 0.000262144 0.000524288)
VIN19 nd19 0 PULSE(0 1.8 0.000262144 20p 20p 0.000524288 0.001048576)
VIN20 nd20 0 PULSE(0 1.8 0.000524288 20p 20p 0.001048576 0.002097152)
VIN21 nd21 0 PULSE(0 1.8 0.001048576 20p 20p 0.002097152 0.004194304)
VIN22 nd22 0 PULSE(0 1.8 0.002097152 20p 20p 0.004194304 0.008388608)
VIN23 nd23 0 PULSE(0 1.8 0.004194304 20p 20p 0.008388608 0.016777216)
VIN24 nd24 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN25 nd25 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN26 nd26 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN27 nd27 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN28 nd28 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN29 nd29 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN30 nd30 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN31 nd31 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN32 nr0 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN33 nr1 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN34 nr2 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN35 nr3 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN36 nr4 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN37 nr5 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN38 nen 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
CT1 t1 0 0.1f
CT2 t2 0 0.1f
CT3 t3 0 0.1f
M1 t1 nd0 vdd vdd pch w=2u l=180n
M2 t1 nd1 vdd vdd pch w=2u l=180n
CT4 t4 0 0.1f
M3 t1 nd0 t4 0 nch w=1u l=180n
M4 t4 nd1 0 0 nch w=1u l=180n
M5 t2 nd0 vdd vdd pch w=2u l=180n
M6 t2 t1 vdd vdd pch w=2u l=180n
CT5 t5 0 0.1f
M7 t2 nd0 t5 0 nch w=1u l=180n
M8 t5 t1 0 0 nch w=1u l=180n
M9 t3 nd1 vdd vdd pch w=2u l=180n
M10 t3 t1 vdd vdd pch w=2u l=180n
CT6 t6 0 0.1f
M11 t3 nd1 t6 0 nch w=1u l=180n
M12 t6 t1 0 0 nch w=1u l=180n
M13 nw1 t2 vdd vdd pch w=2u l=180n
M14 nw1 t3 vdd vdd pch w=2u l=180n
CT7 t7 0 0.1f
M15 nw1 t2 t7 0 nch w=1u l=180n
M16 t7 t3 0 0 nch w=1u l=180n
Cnw1 nw1 0 2f
CT8 t8 0 0.1f
CT9 t9 0 0.1f
CT10 t10 0 0.1f
M17 t8 nw1 vdd vdd pch w=2u l=180n
M18 t8 nd3 vdd vdd pch w=2u l=180n
CT11 t11 0 0.1f
M19 t8 nw1 t11 0 nch w=1u l=180n
M20 t11 nd3 0 0 nch w=1u l=180n
M21 t9 nw1 vdd vdd pch w=2u l=180n
M22 t9 t8 vdd vdd pch w=2u l=180n
CT12 t12 0 0.1f
M23 t9 nw1 t12 0 nch w=1u l=180n
M24 t12 t8 0 0 nch w=1u l=180n
M25 t10 nd3 vdd vdd pch w=2u l=180n
M26 t10 t8 vdd vdd pch w=2u l=180n
CT13 t13 0 0.1f
M27 t10 nd3 t13 0 nch w=1u l=180n
M28 t13 t8 0 0 nch w=1u l=180n
M29 nw2 t9 vdd vdd pch w=2u l=180n
M30 nw2 t10 vdd vdd pch w=2u l=180n
CT14 t14 0 0.1f
M31 nw2 t9 t14 0 nch w=1u l=180n
M32 t14 t10 0 0 nch w=1u l=180n
Cnw2 nw2 0 2f
CT15 t15 0 0.1f
CT16 t16 0 0.1f
CT17 t17 0 0.1f
M33 t15 nw2 vdd vdd pch w=2u l=180n
M34 t15 nd4 vdd vdd pch w=2u l=180n
CT18 t18 0 0.1f
M35 t15 nw2 t18 0 nch w=1u l=180n
M36 t18 nd4 0 0 nch w=1u l=180n
M37 t16 nw2 vdd vdd pch w=2u l=180n
M38 t16 t15 vdd vdd pch w=2u l=180n
CT19 t19 0 0.1f
M39 t16 nw2 t19 0 nch w=1u l=180n
M40 t19 t15 0 0 nch w=1u l=180n
M41 t17 nd4 vdd vdd pch w=2u l=180n
M42 t17 t15 vdd vdd pch w=2u l=180n
CT20 t20 0 0.1f
M43 t17 nd4 t20 0 nch w=1u l=180n
M44 t20 t15 0 0 nch w=1u l=180n
M45 nw3 t16 vdd vdd pch w=2u l=180n
M46 nw3 t17 vdd vdd pch w=2u l=180n
CT21 t21 0 0.1f
M47 nw3 t16 t21 0 nch w=1u l=180n
M48 t21 t17 0 0 nch w=1u l=180n
Cnw3 nw3 0 2f
CT22 t22 0 0.1f
CT23 t23 0 0.1f
CT24 t24 0 0.1f
M49 t22 nw3 vdd vdd pch w=2u l=180n
M50 t22 nd6 vdd vdd pch w=2u l=180n
CT25 t25 0 0.1f
M51 t22 nw3 t25 0 nch w=1u l=180n
M52 t25 nd6 0 0 nch w=1u l=180n
M53 t23 nw3 vdd vdd pch w=2u l=180n
M54 t23 t22 vdd vdd pch w=2u l=180n
CT26 t26 0 0.1f
M55 t23 nw3 t26 0 nch w=1u l=180n
M56 t26 t22 0 0 nch w=1u l=180n
M57 t24 nd6 vdd vdd pch w=2u l=180n
M58 t24 t22 vdd vdd pch w=2u l=180n
CT27 t27 0 0.1f
M59 t24 nd6 t27 0 nch w=1u l=180n
M60 t27 t22 0 0 nch w=1u l=180n
M61 nw4 t23 vdd vdd pch w=2u l=180n
M62 nw4 t24 vdd vdd pch w=2u l=180n
CT28 t28 0 0.1f
M63 nw4 t23 t28 0 nch w=1u l=180n
M64 t28 t24 0 0 nch w=1u l=180n
Cnw4 nw4 0 2f
CT29 t29 0 0.1f
CT30 t30 0 0.1f
CT31 t31 0 0.1f
M65 t29 nw4 vdd vdd pch w=2u l=180n
M66 t29 nd8 vdd vdd pch w=2u l=180n
CT32 t32 0 0.1f
M67 t29 nw4 t32 0 nch w=1u l=180n
M68 t32 nd8 0 0 nch w=1u l=180n
M69 t30 nw4 vdd vdd pch w=2u l=180n
M70 t30 t29 vdd vdd pch w=2u l=180n
CT33 t33 0 0.1f
M71 t30 nw4 t33 0 nch w=1u l=180n
M72 t33 t29 0 0 nch w=1u l=180n
M73 t31 nd8 vdd vdd pch w=2u l=180n
M74 t31 t29 vdd vdd pch w=2u l=180n
CT34 t34 0 0.1f
M75 t31 nd8 t34 0 nch w=1u l=180n
M76 t34 t29 0 0 nch w=1u l=180n
M77 nw5 t30 vdd vdd pch w=2u l=180n
M78 nw5 t31 vdd vdd pch w=2u l=180n
CT35 t35 0 0.1f
M79 nw5 t30 t35 0 nch w=1u l=180n
M80 t35 t31 0 0 nch w=1u l=180n
Cnw5 nw5 0 2f
CT36 t36 0 0.1f
CT37 t37 0 0.1f
CT38 t38 0 0.1f
M81 t36 nw5 vdd vdd pch w=2u l=180n
M82 t36 nd10 vdd vdd pch w=2u l=180n
CT39 t39 0 0.1f
M83 t36 nw5 t39 0 nch w=1u l=180n
M84 t39 nd10 0 0 nch w=1u l=180n
M85 t37 nw5 vdd vdd pch w=2u l=180n
M86 t37 t36 vdd vdd pch w=2u l=180n
CT40 t40 0 0.1f
M87 t37 nw5 t40 0 nch w=1u l=180n
M88 t40 t36 0 0 nch w=1u l=180n
M89 t38 nd10 vdd vdd pch w=2u l=180n
M90 t38 t36 vdd vdd pch w=2u l=180n
CT41 t41 0 0.1f
M91 t38 nd10 t41 0 nch w=1u l=180n
M92 t41 t36 0 0 nch w=1u l=180n
M93 nw6 t37 vdd vdd pch w=2u l=180n
M94 nw6 t38 vdd vdd pch w=2u l=180n
CT42 t42 0 0.1f
M95 nw6 t37 t42 0 nch w=1u l=180n
M96 t42 t38 0 0 nch w=1u l=180n
Cnw6 nw6 0 2f
CT43 t43 0 0.1f
CT44 t44 0 0.1f
CT45 t45 0 0.1f
M97 t43 nw6 vdd vdd pch w=2u l=180n
M98 t43 nd11 vdd vdd pch w=2u l=180n
CT46 t46 0 0.1f
M99 t43 nw6 t46 0 nch w=1u l=180n
M100 t46 nd11 0 0 nch w=1u l=180n
M101 t44 nw6 vdd vdd pch w=2u l=180n
M102 t44 t43 vdd vdd pch w=2u l=180n
CT47 t47 0 0.1f
M103 t44 nw6 t47 0 nch w=1u l=180n
M104 t47 t43 0 0 nch w=1u l=180n
M105 t45 nd11 vdd vdd pch w=2u l=180n
M106 t45 t43 vdd vdd pch w=2u l=180n
CT48 t48 0 0.1f
M107 t45 nd11 t48 0 nch w=1u l=180n
M108 t48 t43 0 0 nch w=1u l=180n
M109 nw7 t44 vdd vdd pch w=2u l=180n
M110 nw7 t45 vdd vdd pch w=2u l=180n
CT49 t49 0 0.1f
M111 nw7 t44 t49 0 nch w=1u l=180n
M112 t49 t45 0 0 nch w=1u l=180n
Cnw7 nw7 0 2f
CT50 t50 0 0.1f
CT51 t51 0 0.1f
CT52 t52 0 0.1f
M113 t50 nw7 vdd vdd pch w=2u l=180n
M114 t50 nd13 vdd vdd pch w=2u l=180n
CT53 t53 0 0.1f
M115 t50 nw7 t53 0 nch w=1u l=180n
M116 t53 nd13 0 0 nch w=1u l=180n
M117 t51 nw7 vdd vdd pch w=2u l=180n
M118 t51 t50 vdd vdd pch w=2u l=180n
CT54 t54 0 0.1f
M119 t51 nw7 t54 0 nch w=1u l=180n
M120 t54 t50 0 0 nch w=1u l=180n
M121 t52 nd13 vdd vdd pch w=2u l=180n
M122 t52 t50 vdd vdd pch w=2u l=180n
CT55 t55 0 0.1f
M123 t52 nd13 t55 0 nch w=1u l=180n
M124 t55 t50 0 0 nch w=1u l=180n
M125 nw8 t51 vdd vdd pch w=2u l=180n
M126 nw8 t52 vdd vdd pch w=2u l=180n
CT56 t56 0 0.1f
M127 nw8 t51 t56 0 nch w=1u l=180n
M128 t56 t52 0 0 nch w=1u l=180n
Cnw8 nw8 0 2f
CT57 t57 0 0.1f
CT58 t58 0 0.1f
CT59 t59 0 0.1f
M129 t57 nw8 vdd vdd pch w=2u l=180n
M130 t57 nd15 vdd vdd pch w=2u l=180n
CT60 t60 0 0.1f
M131 t57 nw8 t60 0 nch w=1u l=180n
M132 t60 nd15 0 0 nch w=1u l=180n
M133 t58 nw8 vdd vdd pch w=2u l=180n
M134 t58 t57 vdd vdd pch w=2u l=180n
CT61 t61 0 0.1f
M135 t58 nw8 t61 0 nch w=1u l=180n
M136 t61 t57 0 0 nch w=1u l=180n
M137 t59 nd15 vdd vdd pch w=2u l=180n
M138 t59 t57 vdd vdd pch w=2u l=180n
CT62 t62 0 0.1f
M139 t59 nd15 t62 0 nch w=1u l=180n
M140 t62 t57 0 0 nch w=1u l=180n
M141 nw9 t58 vdd vdd pch w=2u l=180n
M142 nw9 t59 vdd vdd pch w=2u l=180n
CT63 t63 0 0.1f
M143 nw9 t58 t63 0 nch w=1u l=180n
M144 t63 t59 0 0 nch w=1u l=180n
Cnw9 nw9 0 2f
CT64 t64 0 0.1f
CT65 t65 0 0.1f
CT66 t66 0 0.1f
M145 t64 nw9 vdd vdd pch w=2u l=180n
M146 t64 nd17 vdd vdd pch w=2u l=180n
CT67 t67 0 0.1f
M147 t64 nw9 t67 0 nch w=1u l=180n
M148 t67 nd17 0 0 nch w=1u l=180n
M149 t65 nw9 vdd vdd pch w=2u l=180n
M150 t65 t64 vdd vdd pch w=2u l=180n
CT68 t68 0 0.1f
M151 t65 nw9 t68 0 nch w=1u l=180n
M152 t68 t64 0 0 nch w=1u l=180n
M153 t66 nd17 vdd vdd pch w=2u l=180n
M154 t66 t64 vdd vdd pch w=2u l=180n
CT69 t69 0 0.1f
M155 t66 nd17 t69 0 nch w=1u l=180n
M156 t69 t64 0 0 nch w=1u l=180n
M157 nw10 t65 vdd vdd pch w=2u l=180n
M158 nw10 t66 vdd vdd pch w=2u l=180n
CT70 t70 0 0.1f
M159 nw10 t65 t70 0 nch w=1u l=180n
M160 t70 t66 0 0 nch w=1u l=180n
Cnw10 nw10 0 2f
CT71 t71 0 0.1f
CT72 t72 0 0.1f
CT73 t73 0 0.1f
M161 t71 nw10 vdd vdd pch w=2u l=180n
M162 t71 nd19 vdd vdd pch w=2u l=180n
CT74 t74 0 0.1f
M163 t71 nw10 t74 0 nch w=1u l=180n
M164 t74 nd19 0 0 nch w=1u l=180n
M165 t72 nw10 vdd vdd pch w=2u l=180n
M166 t72 t71 vdd vdd pch w=2u l=180n
CT75 t75 0 0.1f
M167 t72 nw10 t75 0 nch w=1u l=180n
M168 t75 t71 0 0 nch w=1u l=180n
M169 t73 nd19 vdd vdd pch w=2u l=180n
M170 t73 t71 vdd vdd pch w=2u l=180n
CT76 t76 0 0.1f
M171 t73 nd19 t76 0 nch w=1u l=180n
M172 t76 t71 0 0 nch w=1u l=180n
M173 nw11 t72 vdd vdd pch w=2u l=180n
M174 nw11 t73 vdd vdd pch w=2u l=180n
CT77 t77 0 0.1f
M175 nw11 t72 t77 0 nch w=1u l=180n
M176 t77 t73 0 0 nch w=1u l=180n
Cnw11 nw11 0 2f
CT78 t78 0 0.1f
CT79 t79 0 0.1f
CT80 t80 0 0.1f
M177 t78 nw11 vdd vdd pch w=2u l=180n
M178 t78 nd21 vdd vdd pch w=2u l=180n
CT81 t81 0 0.1f
M179 t78 nw11 t81 0 nch w=1u l=180n
M180 t81 nd21 0 0 nch w=1u l=180n
M181 t79 nw11 vdd vdd pch w=2u l=180n
M182 t79 t78 vdd vdd pch w=2u l=180n
CT82 t82 0 0.1f
M183 t79 nw11 t82 0 nch w=1u l=180n
M184 t82 t78 0 0 nch w=1u l=180n
M185 t80 nd21 vdd vdd pch w=2u l=180n
M186 t80 t78 vdd vdd pch w=2u l=180n
CT83 t83 0 0.1f
M187 t80 nd21 t83 0 nch w=1u l=180n
M188 t83 t78 0 0 nch w=1u l=180n
M189 nw12 t79 vdd vdd pch w=2u l=180n
M190 nw12 t80 vdd vdd pch w=2u l=180n
CT84 t84 0 0.1f
M191 nw12 t79 t84 0 nch w=1u l=180n
M192 t84 t80 0 0 nch w=1u l=180n
Cnw12 nw12 0 2f
CT85 t85 0 0.1f
CT86 t86 0 0.1f
CT87 t87 0 0.1f
M193 t85 nw12 vdd vdd pch w=2u l=180n
M194 t85 nd23 vdd vdd pch w=2u l=180n
CT88 t88 0 0.1f
M195 t85 nw12 t88 0 nch w=1u l=180n
M196 t88 nd23 0 0 nch w=1u l=180n
M197 t86 nw12 vdd vdd pch w=2u l=180n
M198 t86 t85 vdd vdd pch w=2u l=180n
CT89 t89 0 0.1f
M199 t86 nw12 t89 0 nch w=1u l=180n
M200 t89 t85 0 0 nch w=1u l=180n
M201 t87 nd23 vdd vdd pch w=2u l=180n
M202 t87 t85 vdd vdd pch w=2u l=180n
CT90 t90 0 0.1f
M203 t87 nd23 t90 0 nch w=1u l=180n
M204 t90 t85 0 0 nch w=1u l=180n
M205 nw13 t86 vdd vdd pch w=2u l=180n
M206 nw13 t87 vdd vdd pch w=2u l=180n
CT91 t91 0 0.1f
M207 nw13 t86 t91 0 nch w=1u l=180n
M208 t91 t87 0 0 nch w=1u l=180n
Cnw13 nw13 0 2f
CT92 t92 0 0.1f
CT93 t93 0 0.1f
CT94 t94 0 0.1f
M209 t92 nw13 vdd vdd pch w=2u l=180n
M210 t92 nd25 vdd vdd pch w=2u l=180n
CT95 t95 0 0.1f
M211 t92 nw13 t95 0 nch w=1u l=180n
M212 t95 nd25 0 0 nch w=1u l=180n
M213 t93 nw13 vdd vdd pch w=2u l=180n
M214 t93 t92 vdd vdd pch w=2u l=180n
CT96 t96 0 0.1f
M215 t93 nw13 t96 0 nch w=1u l=180n
M216 t96 t92 0 0 nch w=1u l=180n
M217 t94 nd25 vdd vdd pch w=2u l=180n
M218 t94 t92 vdd vdd pch w=2u l=180n
CT97 t97 0 0.1f
M219 t94 nd25 t97 0 nch w=1u l=180n
M220 t97 t92 0 0 nch w=1u l=180n
M221 nw14 t93 vdd vdd pch w=2u l=180n
M222 nw14 t94 vdd vdd pch w=2u l=180n
CT98 t98 0 0.1f
M223 nw14 t93 t98 0 nch w=1u l=180n
M224 t98 t94 0 0 nch w=1u l=180n
Cnw14 nw14 0 2f
CT99 t99 0 0.1f
CT100 t100 0 0.1f
CT101 t101 0 0.1f
M225 t99 nw14 vdd vdd pch w=2u l=180n
M226 t99 nd26 vdd vdd pch w=2u l=180n
CT102 t102 0 0.1f
M227 t99 nw14 t102 0 nch w=1u l=180n
M228 t102 nd26 0 0 nch w=1u l=180n
M229 t100 nw14 vdd vdd pch w=2u l=180n
M230 t100 t99 vdd vdd pch w=2u l=180n
CT103 t103 0 0.1f
M231 t100 nw14 t103 0 nch w=1u l=180n
M232 t103 t99 0 0 nch w=1u l=180n
M233 t101 nd26 vdd vdd pch w=2u l=180n
M234 t101 t99 vdd vdd pch w=2u l=180n
CT104 t104 0 0.1f
M235 t101 nd26 t104 0 nch w=1u l=180n
M236 t104 t99 0 0 nch w=1u l=180n
M237 nw15 t100 vdd vdd pch w=2u l=180n
M238 nw15 t101 vdd vdd pch w=2u l=180n
CT105 t105 0 0.1f
M239 nw15 t100 t105 0 nch w=1u l=180n
M240 t105 t101 0 0 nch w=1u l=180n
Cnw15 nw15 0 2f
CT106 t106 0 0.1f
CT107 t107 0 0.1f
CT108 t108 0 0.1f
M241 t106 nw15 vdd vdd pch w=2u l=180n
M242 t106 nd28 vdd vdd pch w=2u l=180n
CT109 t109 0 0.1f
M243 t106 nw15 t109 0 nch w=1u l=180n
M244 t109 nd28 0 0 nch w=1u l=180n
M245 t107 nw15 vdd vdd pch w=2u l=180n
M246 t107 t106 vdd vdd pch w=2u l=180n
CT110 t110 0 0.1f
M247 t107 nw15 t110 0 nch w=1u l=180n
M248 t110 t106 0 0 nch w=1u l=180n
M249 t108 nd28 vdd vdd pch w=2u l=180n
M250 t108 t106 vdd vdd pch w=2u l=180n
CT111 t111 0 0.1f
M251 t108 nd28 t111 0 nch w=1u l=180n
M252 t111 t106 0 0 nch w=1u l=180n
M253 nw16 t107 vdd vdd pch w=2u l=180n
M254 nw16 t108 vdd vdd pch w=2u l=180n
CT112 t112 0 0.1f
M255 nw16 t107 t112 0 nch w=1u l=180n
M256 t112 t108 0 0 nch w=1u l=180n
Cnw16 nw16 0 2f
CT113 t113 0 0.1f
CT114 t114 0 0.1f
CT115 t115 0 0.1f
M257 t113 nw16 vdd vdd pch w=2u l=180n
M258 t113 nd30 vdd vdd pch w=2u l=180n
CT116 t116 0 0.1f
M259 t113 nw16 t116 0 nch w=1u l=180n
M260 t116 nd30 0 0 nch w=1u l=180n
M261 t114 nw16 vdd vdd pch w=2u l=180n
M262 t114 t113 vdd vdd pch w=2u l=180n
CT117 t117 0 0.1f
M263 t114 nw16 t117 0 nch w=1u l=180n
M264 t117 t113 0 0 nch w=1u l=180n
M265 t115 nd30 vdd vdd pch w=2u l=180n
M266 t115 t113 vdd vdd pch w=2u l=180n
CT118 t118 0 0.1f
M267 t115 nd30 t118 0 nch w=1u l=180n
M268 t118 t113 0 0 nch w=1u l=180n
M269 nw17 t114 vdd vdd pch w=2u l=180n
M270 nw17 t115 vdd vdd pch w=2u l=180n
CT119 t119 0 0.1f
M271 nw17 t114 t119 0 nch w=1u l=180n
M272 t119 t115 0 0 nch w=1u l=180n
Cnw17 nw17 0 2f
CT120 t120 0 0.1f
CT121 t121 0 0.1f
CT122 t122 0 0.1f
M273 t120 nw17 vdd vdd pch w=2u l=180n
M274 t120 nr0 vdd vdd pch w=2u l=180n
CT123 t123 0 0.1f
M275 t120 nw17 t123 0 nch w=1u l=180n
M276 t123 nr0 0 0 nch w=1u l=180n
M277 t121 nw17 vdd vdd pch w=2u l=180n
M278 t121 t120 vdd vdd pch w=2u l=180n
CT124 t124 0 0.1f
M279 t121 nw17 t124 0 nch w=1u l=180n
M280 t124 t120 0 0 nch w=1u l=180n
M281 t122 nr0 vdd vdd pch w=2u l=180n
M282 t122 t120 vdd vdd pch w=2u l=180n
CT125 t125 0 0.1f
M283 t122 nr0 t125 0 nch w=1u l=180n
M284 t125 t120 0 0 nch w=1u l=180n
M285 nw18 t121 vdd vdd pch w=2u l=180n
M286 nw18 t122 vdd vdd pch w=2u l=180n
CT126 t126 0 0.1f
M287 nw18 t121 t126 0 nch w=1u l=180n
M288 t126 t122 0 0 nch w=1u l=180n
Cnw18 nw18 0 2f
CT127 t127 0 0.1f
CT128 t128 0 0.1f
CT129 t129 0 0.1f
M289 t127 nd0 vdd vdd pch w=2u l=180n
M290 t127 nd2 vdd vdd pch w=2u l=180n
CT130 t130 0 0.1f
M291 t127 nd0 t130 0 nch w=1u l=180n
M292 t130 nd2 0 0 nch w=1u l=180n
M293 t128 nd0 vdd vdd pch w=2u l=180n
M294 t128 t127 vdd vdd pch w=2u l=180n
CT131 t131 0 0.1f
M295 t128 nd0 t131 0 nch w=1u l=180n
M296 t131 t127 0 0 nch w=1u l=180n
M297 t129 nd2 vdd vdd pch w=2u l=180n
M298 t129 t127 vdd vdd pch w=2u l=180n
CT132 t132 0 0.1f
M299 t129 nd2 t132 0 nch w=1u l=180n
M300 t132 t127 0 0 nch w=1u l=180n
M301 nw19 t128 vdd vdd pch w=2u l=180n
M302 nw19 t129 vdd vdd pch w=2u l=180n
CT133 t133 0 0.1f
M303 nw19 t128 t133 0 nch w=1u l=180n
M304 t133 t129 0 0 nch w=1u l=180n
Cnw19 nw19 0 2f
CT134 t134 0 0.1f
CT135 t135 0 0.1f
CT136 t136 0 0.1f
M305 t134 nw19 vdd vdd pch w=2u l=180n
M306 t134 nd3 vdd vdd pch w=2u l=180n
CT137 t137 0 0.1f
M307 t134 nw19 t137 0 nch w=1u l=180n
M308 t137 nd3 0 0 nch w=1u l=180n
M309 t135 nw19 vdd vdd pch w=2u l=180n
M310 t135 t134 vdd vdd pch w=2u l=180n
CT138 t138 0 0.1f
M311 t135 nw19 t138 0 nch w=1u l=180n
M312 t138 t134 0 0 nch w=1u l=180n
M313 t136 nd3 vdd vdd pch w=2u l=180n
M314 t136 t134 vdd vdd pch w=2u l=180n
CT139 t139 0 0.1f
M315 t136 nd3 t139 0 nch w=1u l=180n
M316 t139 t134 0 0 nch w=1u l=180n
M317 nw20 t135 vdd vdd pch w=2u l=180n
M318 nw20 t136 vdd vdd pch w=2u l=180n
CT140 t140 0 0.1f
M319 nw20 t135 t140 0 nch w=1u l=180n
M320 t140 t136 0 0 nch w=1u l=180n
Cnw20 nw20 0 2f
CT141 t141 0 0.1f
CT142 t142 0 0.1f
CT143 t143 0 0.1f
M321 t141 nw20 vdd vdd pch w=2u l=180n
M322 t141 nd5 vdd vdd pch w=2u l=180n
CT144 t144 0 0.1f
M323 t141 nw20 t144 0 nch w=1u l=180n
M324 t144 nd5 0 0 nch w=1u l=180n
M325 t142 nw20 vdd vdd pch w=2u l=180n
M326 t142 t141 vdd vdd pch w=2u l=180n
CT145 t145 0 0.1f
M327 t142 nw20 t145 0 nch w=1u l=180n
M328 t145 t141 0 0 nch w=1u l=180n
M329 t143 nd5 vdd vdd pch w=2u l=180n
M330 t143 t141 vdd vdd pch w=2u l=180n
CT146 t146 0 0.1f
M331 t143 nd5 t146 0 nch w=1u l=180n
M332 t146 t141 0 0 nch w=1u l=180n
M333 nw21 t142 vdd vdd pch w=2u l=180n
M334 nw21 t143 vdd vdd pch w=2u l=180n
CT147 t147 0 0.1f
M335 nw21 t142 t147 0 nch w=1u l=180n
M336 t147 t143 0 0 nch w=1u l=180n
Cnw21 nw21 0 2f
CT148 t148 0 0.1f
CT149 t149 0 0.1f
CT150 t150 0 0.1f
M337 t148 nw21 vdd vdd pch w=2u l=180n
M338 t148 nd6 vdd vdd pch w=2u l=180n
CT151 t151 0 0.1f
M339 t148 nw21 t151 0 nch w=1u l=180n
M340 t151 nd6 0 0 nch w=1u l=180n
M341 t149 nw21 vdd vdd pch w=2u l=180n
M342 t149 t148 vdd vdd pch w=2u l=180n
CT152 t152 0 0.1f
M343 t149 nw21 t152 0 nch w=1u l=180n
M344 t152 t148 0 0 nch w=1u l=180n
M345 t150 nd6 vdd vdd pch w=2u l=180n
M346 t150 t148 vdd vdd pch w=2u l=180n
CT153 t153 0 0.1f
M347 t150 nd6 t153 0 nch w=1u l=180n
M348 t153 t148 0 0 nch w=1u l=180n
M349 nw22 t149 vdd vdd pch w=2u l=180n
M350 nw22 t150 vdd vdd pch w=2u l=180n
CT154 t154 0 0.1f
M351 nw22 t149 t154 0 nch w=1u l=180n
M352 t154 t150 0 0 nch w=1u l=180n
Cnw22 nw22 0 2f
CT155 t155 0 0.1f
CT156 t156 0 0.1f
CT157 t157 0 0.1f
M353 t155 nw22 vdd vdd pch w=2u l=180n
M354 t155 nd9 vdd vdd pch w=2u l=180n
CT158 t158 0 0.1f
M355 t155 nw22 t158 0 nch w=1u l=180n
M356 t158 nd9 0 0 nch w=1u l=180n
M357 t156 nw22 vdd vdd pch w=2u l=180n
M358 t156 t155 vdd vdd pch w=2u l=180n
CT159 t159 0 0.1f
M359 t156 nw22 t159 0 nch w=1u l=180n
M360 t159 t155 0 0 nch w=1u l=180n
M361 t157 nd9 vdd vdd pch w=2u l=180n
M362 t157 t155 vdd vdd pch w=2u l=180n
CT160 t160 0 0.1f
M363 t157 nd9 t160 0 nch w=1u l=180n
M364 t160 t155 0 0 nch w=1u l=180n
M365 nw23 t156 vdd vdd pch w=2u l=180n
M366 nw23 t157 vdd vdd pch w=2u l=180n
CT161 t161 0 0.1f
M367 nw23 t156 t161 0 nch w=1u l=180n
M368 t161 t157 0 0 nch w=1u l=180n
Cnw23 nw23 0 2f
CT162 t162 0 0.1f
CT163 t163 0 0.1f
CT164 t164 0 0.1f
M369 t162 nw23 vdd vdd pch w=2u l=180n
M370 t162 nd10 vdd vdd pch w=2u l=180n
CT165 t165 0 0.1f
M371 t162 nw23 t165 0 nch w=1u l=180n
M372 t165 nd10 0 0 nch w=1u l=180n
M373 t163 nw23 vdd vdd pch w=2u l=180n
M374 t163 t162 vdd vdd pch w=2u l=180n
CT166 t166 0 0.1f
M375 t163 nw23 t166 0 nch w=1u l=180n
M376 t166 t162 0 0 nch w=1u l=180n
M377 t164 nd10 vdd vdd pch w=2u l=180n
M378 t164 t162 vdd vdd pch w=2u l=180n
CT167 t167 0 0.1f
M379 t164 nd10 t167 0 nch w=1u l=180n
M380 t167 t162 0 0 nch w=1u l=180n
M381 nw24 t163 vdd vdd pch w=2u l=180n
M382 nw24 t164 vdd vdd pch w=2u l=180n
CT168 t168 0 0.1f
M383 nw24 t163 t168 0 nch w=1u l=180n
M384 t168 t164 0 0 nch w=1u l=180n
Cnw24 nw24 0 2f
CT169 t169 0 0.1f
CT170 t170 0 0.1f
CT171 t171 0 0.1f
M385 t169 nw24 vdd vdd pch w=2u l=180n
M386 t169 nd12 vdd vdd pch w=2u l=180n
CT172 t172 0 0.1f
M387 t169 nw24 t172 0 nch w=1u l=180n
M388 t172 nd12 0 0 nch w=1u l=180n
M389 t170 nw24 vdd vdd pch w=2u l=180n
M390 t170 t169 vdd vdd pch w=2u l=180n
CT173 t173 0 0.1f
M391 t170 nw24 t173 0 nch w=1u l=180n
M392 t173 t169 0 0 nch w=1u l=180n
M393 t171 nd12 vdd vdd pch w=2u l=180n
M394 t171 t169 vdd vdd pch w=2u l=180n
CT174 t174 0 0.1f
M395 t171 nd12 t174 0 nch w=1u l=180n
M396 t174 t169 0 0 nch w=1u l=180n
M397 nw25 t170 vdd vdd pch w=2u l=180n
M398 nw25 t171 vdd vdd pch w=2u l=180n
CT175 t175 0 0.1f
M399 nw25 t170 t175 0 nch w=1u l=180n
M400 t175 t171 0 0 nch w=1u l=180n
Cnw25 nw25 0 2f
CT176 t176 0 0.1f
CT177 t177 0 0.1f
CT178 t178 0 0.1f
M401 t176 nw25 vdd vdd pch w=2u l=180n
M402 t176 nd13 vdd vdd pch w=2u l=180n
CT179 t179 0 0.1f
M403 t176 nw25 t179 0 nch w=1u l=180n
M404 t179 nd13 0 0 nch w=1u l=180n
M405 t177 nw25 vdd vdd pch w=2u l=180n
M406 t177 t176 vdd vdd pch w=2u l=180n
CT180 t180 0 0.1f
M407 t177 nw25 t180 0 nch w=1u l=180n
M408 t180 t176 0 0 nch w=1u l=180n
M409 t178 nd13 vdd vdd pch w=2u l=180n
M410 t178 t176 vdd vdd pch w=2u l=180n
CT181 t181 0 0.1f
M411 t178 nd13 t181 0 nch w=1u l=180n
M412 t181 t176 0 0 nch w=1u l=180n
M413 nw26 t177 vdd vdd pch w=2u l=180n
M414 nw26 t178 vdd vdd pch w=2u l=180n
CT182 t182 0 0.1f
M415 nw26 t177 t182 0 nch w=1u l=180n
M416 t182 t178 0 0 nch w=1u l=180n
Cnw26 nw26 0 2f
CT183 t183 0 0.1f
CT184 t184 0 0.1f
CT185 t185 0 0.1f
M417 t183 nw26 vdd vdd pch w=2u l=180n
M418 t183 nd16 vdd vdd pch w=2u l=180n
CT186 t186 0 0.1f
M419 t183 nw26 t186 0 nch w=1u l=180n
M420 t186 nd16 0 0 nch w=1u l=180n
M421 t184 nw26 vdd vdd pch w=2u l=180n
M422 t184 t183 vdd vdd pch w=2u l=180n
CT187 t187 0 0.1f
M423 t184 nw26 t187 0 nch w=1u l=180n
M424 t187 t183 0 0 nch w=1u l=180n
M425 t185 nd16 vdd vdd pch w=2u l=180n
M426 t185 t183 vdd vdd pch w=2u l=180n
CT188 t188 0 0.1f
M427 t185 nd16 t188 0 nch w=1u l=180n
M428 t188 t183 0 0 nch w=1u l=180n
M429 nw27 t184 vdd vdd pch w=2u l=180n
M430 nw27 t185 vdd vdd pch w=2u l=180n
CT189 t189 0 0.1f
M431 nw27 t184 t189 0 nch w=1u l=180n
M432 t189 t185 0 0 nch w=1u l=180n
Cnw27 nw27 0 2f
CT190 t190 0 0.1f
CT191 t191 0 0.1f
CT192 t192 0 0.1f
M433 t190 nw27 vdd vdd pch w=2u l=180n
M434 t190 nd17 vdd vdd pch w=2u l=180n
CT193 t193 0 0.1f
M435 t190 nw27 t193 0 nch w=1u l=180n
M436 t193 nd17 0 0 nch w=1u l=180n
M437 t191 nw27 vdd vdd pch w=2u l=180n
M438 t191 t190 vdd vdd pch w=2u l=180n
CT194 t194 0 0.1f
M439 t191 nw27 t194 0 nch w=1u l=180n
M440 t194 t190 0 0 nch w=1u l=180n
M441 t192 nd17 vdd vdd pch w=2u l=180n
M442 t192 t190 vdd vdd pch w=2u l=180n
CT195 t195 0 0.1f
M443 t192 nd17 t195 0 nch w=1u l=180n
M444 t195 t190 0 0 nch w=1u l=180n
M445 nw28 t191 vdd vdd pch w=2u l=180n
M446 nw28 t192 vdd vdd pch w=2u l=180n
CT196 t196 0 0.1f
M447 nw28 t191 t196 0 nch w=1u l=180n
M448 t196 t192 0 0 nch w=1u l=180n
Cnw28 nw28 0 2f
CT197 t197 0 0.1f
CT198 t198 0 0.1f
CT199 t199 0 0.1f
M449 t197 nw28 vdd vdd pch w=2u l=180n
M450 t197 nd20 vdd vdd pch w=2u l=180n
CT200 t200 0 0.1f
M451 t197 nw28 t200 0 nch w=1u l=180n
M452 t200 nd20 0 0 nch w=1u l=180n
M453 t198 nw28 vdd vdd pch w=2u l=180n
M454 t198 t197 vdd vdd pch w=2u l=180n
CT201 t201 0 0.1f
M455 t198 nw28 t201 0 nch w=1u l=180n
M456 t201 t197 0 0 nch w=1u l=180n
M457 t199 nd20 vdd vdd pch w=2u l=180n
M458 t199 t197 vdd vdd pch w=2u l=180n
CT202 t202 0 0.1f
M459 t199 nd20 t202 0 nch w=1u l=180n
M460 t202 t197 0 0 nch w=1u l=180n
M461 nw29 t198 vdd vdd pch w=2u l=180n
M462 nw29 t199 vdd vdd pch w=2u l=180n
CT203 t203 0 0.1f
M463 nw29 t198 t203 0 nch w=1u l=180n
M464 t203 t199 0 0 nch w=1u l=180n
Cnw29 nw29 0 2f
CT204 t204 0 0.1f
CT205 t205 0 0.1f
CT206 t206 0 0.1f
M465 t204 nw29 vdd vdd pch w=2u l=180n
M466 t204 nd21 vdd vdd pch w=2u l=180n
CT207 t207 0 0.1f
M467 t204 nw29 t207 0 nch w=1u l=180n
M468 t207 nd21 0 0 nch w=1u l=180n
M469 t205 nw29 vdd vdd pch w=2u l=180n
M470 t205 t204 vdd vdd pch w=2u l=180n
CT208 t208 0 0.1f
M471 t205 nw29 t208 0 nch w=1u l=180n
M472 t208 t204 0 0 nch w=1u l=180n
M473 t206 nd21 vdd vdd pch w=2u l=180n
M474 t206 t204 vdd vdd pch w=2u l=180n
CT209 t209 0 0.1f
M475 t206 nd21 t209 0 nch w=1u l=180n
M476 t209 t204 0 0 nch w=1u l=180n
M477 nw30 t205 vdd vdd pch w=2u l=180n
M478 nw30 t206 vdd vdd pch w=2u l=180n
CT210 t210 0 0.1f
M479 nw30 t205 t210 0 nch w=1u l=180n
M480 t210 t206 0 0 nch w=1u l=180n
Cnw30 nw30 0 2f
CT211 t211 0 0.1f
CT212 t212 0 0.1f
CT213 t213 0 0.1f
M481 t211 nw30 vdd vdd pch w=2u l=180n
M482 t211 nd24 vdd vdd pch w=2u l=180n
CT214 t214 0 0.1f
M483 t211 nw30 t214 0 nch w=1u l=180n
M484 t214 nd24 0 0 nch w=1u l=180n
M485 t212 nw30 vdd vdd pch w=2u l=180n
M486 t212 t211 vdd vdd pch w=2u l=180n
CT215 t215 0 0.1f
M487 t212 nw30 t215 0 nch w=1u l=180n
M488 t215 t211 0 0 nch w=1u l=180n
M489 t213 nd24 vdd vdd pch w=2u l=180n
M490 t213 t211 vdd vdd pch w=2u l=180n
CT216 t216 0 0.1f
M491 t213 nd24 t216 0 nch w=1u l=180n
M492 t216 t211 0 0 nch w=1u l=180n
M493 nw31 t212 vdd vdd pch w=2u l=180n
M494 nw31 t213 vdd vdd pch w=2u l=180n
CT217 t217 0 0.1f
M495 nw31 t212 t217 0 nch w=1u l=180n
M496 t217 t213 0 0 nch w=1u l=180n
Cnw31 nw31 0 2f
CT218 t218 0 0.1f
CT219 t219 0 0.1f
CT220 t220 0 0.1f
M497 t218 nw31 vdd vdd pch w=2u l=180n
M498 t218 nd25 vdd vdd pch w=2u l=180n
CT221 t221 0 0.1f
M499 t218 nw31 t221 0 nch w=1u l=180n
M500 t221 nd25 0 0 nch w=1u l=180n
M501 t219 nw31 vdd vdd pch w=2u l=180n
M502 t219 t218 vdd vdd pch w=2u l=180n
CT222 t222 0 0.1f
M503 t219 nw31 t222 0 nch w=1u l=180n
M504 t222 t218 0 0 nch w=1u l=180n
M505 t220 nd25 vdd vdd pch w=2u l=180n
M506 t220 t218 vdd vdd pch w=2u l=180n
CT223 t223 0 0.1f
M507 t220 nd25 t223 0 nch w=1u l=180n
M508 t223 t218 0 0 nch w=1u l=180n
M509 nw32 t219 vdd vdd pch w=2u l=180n
M510 nw32 t220 vdd vdd pch w=2u l=180n
CT224 t224 0 0.1f
M511 nw32 t219 t224 0 nch w=1u l=180n
M512 t224 t220 0 0 nch w=1u l=180n
Cnw32 nw32 0 2f
CT225 t225 0 0.1f
CT226 t226 0 0.1f
CT227 t227 0 0.1f
M513 t225 nw32 vdd vdd pch w=2u l=180n
M514 t225 nd27 vdd vdd pch w=2u l=180n
CT228 t228 0 0.1f
M515 t225 nw32 t228 0 nch w=1u l=180n
M516 t228 nd27 0 0 nch w=1u l=180n
M517 t226 nw32 vdd vdd pch w=2u l=180n
M518 t226 t225 vdd vdd pch w=2u l=180n
CT229 t229 0 0.1f
M519 t226 nw32 t229 0 nch w=1u l=180n
M520 t229 t225 0 0 nch w=1u l=180n
M521 t227 nd27 vdd vdd pch w=2u l=180n
M522 t227 t225 vdd vdd pch w=2u l=180n
CT230 t230 0 0.1f
M523 t227 nd27 t230 0 nch w=1u l=180n
M524 t230 t225 0 0 nch w=1u l=180n
M525 nw33 t226 vdd vdd pch w=2u l=180n
M526 nw33 t227 vdd vdd pch w=2u l=180n
CT231 t231 0 0.1f
M527 nw33 t226 t231 0 nch w=1u l=180n
M528 t231 t227 0 0 nch w=1u l=180n
Cnw33 nw33 0 2f
CT232 t232 0 0.1f
CT233 t233 0 0.1f
CT234 t234 0 0.1f
M529 t232 nw33 vdd vdd pch w=2u l=180n
M530 t232 nd28 vdd vdd pch w=2u l=180n
CT235 t235 0 0.1f
M531 t232 nw33 t235 0 nch w=1u l=180n
M532 t235 nd28 0 0 nch w=1u l=180n
M533 t233 nw33 vdd vdd pch w=2u l=180n
M534 t233 t232 vdd vdd pch w=2u l=180n
CT236 t236 0 0.1f
M535 t233 nw33 t236 0 nch w=1u l=180n
M536 t236 t232 0 0 nch w=1u l=180n
M537 t234 nd28 vdd vdd pch w=2u l=180n
M538 t234 t232 vdd vdd pch w=2u l=180n
CT237 t237 0 0.1f
M539 t234 nd28 t237 0 nch w=1u l=180n
M540 t237 t232 0 0 nch w=1u l=180n
M541 nw34 t233 vdd vdd pch w=2u l=180n
M542 nw34 t234 vdd vdd pch w=2u l=180n
CT238 t238 0 0.1f
M543 nw34 t233 t238 0 nch w=1u l=180n
M544 t238 t234 0 0 nch w=1u l=180n
Cnw34 nw34 0 2f
CT239 t239 0 0.1f
CT240 t240 0 0.1f
CT241 t241 0 0.1f
M545 t239 nw34 vdd vdd pch w=2u l=180n
M546 t239 nd31 vdd vdd pch w=2u l=180n
CT242 t242 0 0.1f
M547 t239 nw34 t242 0 nch w=1u l=180n
M548 t242 nd31 0 0 nch w=1u l=180n
M549 t240 nw34 vdd vdd pch w=2u l=180n
M550 t240 t239 vdd vdd pch w=2u l=180n
CT243 t243 0 0.1f
M551 t240 nw34 t243 0 nch w=1u l=180n
M552 t243 t239 0 0 nch w=1u l=180n
M553 t241 nd31 vdd vdd pch w=2u l=180n
M554 t241 t239 vdd vdd pch w=2u l=180n
CT244 t244 0 0.1f
M555 t241 nd31 t244 0 nch w=1u l=180n
M556 t244 t239 0 0 nch w=1u l=180n
M557 nw35 t240 vdd vdd pch w=2u l=180n
M558 nw35 t241 vdd vdd pch w=2u l=180n
CT245 t245 0 0.1f
M559 nw35 t240 t245 0 nch w=1u l=180n
M560 t245 t241 0 0 nch w=1u l=180n
Cnw35 nw35 0 2f
CT246 t246 0 0.1f
CT247 t247 0 0.1f
CT248 t248 0 0.1f
M561 t246 nw35 vdd vdd pch w=2u l=180n
M562 t246 nr1 vdd vdd pch w=2u l=180n
CT249 t249 0 0.1f
M563 t246 nw35 t249 0 nch w=1u l=180n
M564 t249 nr1 0 0 nch w=1u l=180n
M565 t247 nw35 vdd vdd pch w=2u l=180n
M566 t247 t246 vdd vdd pch w=2u l=180n
CT250 t250 0 0.1f
M567 t247 nw35 t250 0 nch w=1u l=180n
M568 t250 t246 0 0 nch w=1u l=180n
M569 t248 nr1 vdd vdd pch w=2u l=180n
M570 t248 t246 vdd vdd pch w=2u l=180n
CT251 t251 0 0.1f
M571 t248 nr1 t251 0 nch w=1u l=180n
M572 t251 t246 0 0 nch w=1u l=180n
M573 nw36 t247 vdd vdd pch w=2u l=180n
M574 nw36 t248 vdd vdd pch w=2u l=180n
CT252 t252 0 0.1f
M575 nw36 t247 t252 0 nch w=1u l=180n
M576 t252 t248 0 0 nch w=1u l=180n
Cnw36 nw36 0 2f
CT253 t253 0 0.1f
CT254 t254 0 0.1f
CT255 t255 0 0.1f
M577 t253 nd1 vdd vdd pch w=2u l=180n
M578 t253 nd2 vdd vdd pch w=2u l=180n
CT256 t256 0 0.1f
M579 t253 nd1 t256 0 nch w=1u l=180n
M580 t256 nd2 0 0 nch w=1u l=180n
M581 t254 nd1 vdd vdd pch w=2u l=180n
M582 t254 t253 vdd vdd pch w=2u l=180n
CT257 t257 0 0.1f
M583 t254 nd1 t257 0 nch w=1u l=180n
M584 t257 t253 0 0 nch w=1u l=180n
M585 t255 nd2 vdd vdd pch w=2u l=180n
M586 t255 t253 vdd vdd pch w=2u l=180n
CT258 t258 0 0.1f
M587 t255 nd2 t258 0 nch w=1u l=180n
M588 t258 t253 0 0 nch w=1u l=180n
M589 nw37 t254 vdd vdd pch w=2u l=180n
M590 nw37 t255 vdd vdd pch w=2u l=180n
CT259 t259 0 0.1f
M591 nw37 t254 t259 0 nch w=1u l=180n
M592 t259 t255 0 0 nch w=1u l=180n
Cnw37 nw37 0 2f
CT260 t260 0 0.1f
CT261 t261 0 0.1f
CT262 t262 0 0.1f
M593 t260 nw37 vdd vdd pch w=2u l=180n
M594 t260 nd3 vdd vdd pch w=2u l=180n
CT263 t263 0 0.1f
M595 t260 nw37 t263 0 nch w=1u l=180n
M596 t263 nd3 0 0 nch w=1u l=180n
M597 t261 nw37 vdd vdd pch w=2u l=180n
M598 t261 t260 vdd vdd pch w=2u l=180n
CT264 t264 0 0.1f
M599 t261 nw37 t264 0 nch w=1u l=180n
M600 t264 t260 0 0 nch w=1u l=180n
M601 t262 nd3 vdd vdd pch w=2u l=180n
M602 t262 t260 vdd vdd pch w=2u l=180n
CT265 t265 0 0.1f
M603 t262 nd3 t265 0 nch w=1u l=180n
M604 t265 t260 0 0 nch w=1u l=180n
M605 nw38 t261 vdd vdd pch w=2u l=180n
M606 nw38 t262 vdd vdd pch w=2u l=180n
CT266 t266 0 0.1f
M607 nw38 t261 t266 0 nch w=1u l=180n
M608 t266 t262 0 0 nch w=1u l=180n
Cnw38 nw38 0 2f
CT267 t267 0 0.1f
CT268 t268 0 0.1f
CT269 t269 0 0.1f
M609 t267 nw38 vdd vdd pch w=2u l=180n
M610 t267 nd7 vdd vdd pch w=2u l=180n
CT270 t270 0 0.1f
M611 t267 nw38 t270 0 nch w=1u l=180n
M612 t270 nd7 0 0 nch w=1u l=180n
M613 t268 nw38 vdd vdd pch w=2u l=180n
M614 t268 t267 vdd vdd pch w=2u l=180n
CT271 t271 0 0.1f
M615 t268 nw38 t271 0 nch w=1u l=180n
M616 t271 t267 0 0 nch w=1u l=180n
M617 t269 nd7 vdd vdd pch w=2u l=180n
M618 t269 t267 vdd vdd pch w=2u l=180n
CT272 t272 0 0.1f
M619 t269 nd7 t272 0 nch w=1u l=180n
M620 t272 t267 0 0 nch w=1u l=180n
M621 nw39 t268 vdd vdd pch w=2u l=180n
M622 nw39 t269 vdd vdd pch w=2u l=180n
CT273 t273 0 0.1f
M623 nw39 t268 t273 0 nch w=1u l=180n
M624 t273 t269 0 0 nch w=1u l=180n
Cnw39 nw39 0 2f
CT274 t274 0 0.1f
CT275 t275 0 0.1f
CT276 t276 0 0.1f
M625 t274 nw39 vdd vdd pch w=2u l=180n
M626 t274 nd8 vdd vdd pch w=2u l=180n
CT277 t277 0 0.1f
M627 t274 nw39 t277 0 nch w=1u l=180n
M628 t277 nd8 0 0 nch w=1u l=180n
M629 t275 nw39 vdd vdd pch w=2u l=180n
M630 t275 t274 vdd vdd pch w=2u l=180n
CT278 t278 0 0.1f
M631 t275 nw39 t278 0 nch w=1u l=180n
M632 t278 t274 0 0 nch w=1u l=180n
M633 t276 nd8 vdd vdd pch w=2u l=180n
M634 t276 t274 vdd vdd pch w=2u l=180n
CT279 t279 0 0.1f
M635 t276 nd8 t279 0 nch w=1u l=180n
M636 t279 t274 0 0 nch w=1u l=180n
M637 nw40 t275 vdd vdd pch w=2u l=180n
M638 nw40 t276 vdd vdd pch w=2u l=180n
CT280 t280 0 0.1f
M639 nw40 t275 t280 0 nch w=1u l=180n
M640 t280 t276 0 0 nch w=1u l=180n
Cnw40 nw40 0 2f
CT281 t281 0 0.1f
CT282 t282 0 0.1f
CT283 t283 0 0.1f
M641 t281 nw40 vdd vdd pch w=2u l=180n
M642 t281 nd9 vdd vdd pch w=2u l=180n
CT284 t284 0 0.1f
M643 t281 nw40 t284 0 nch w=1u l=180n
M644 t284 nd9 0 0 nch w=1u l=180n
M645 t282 nw40 vdd vdd pch w=2u l=180n
M646 t282 t281 vdd vdd pch w=2u l=180n
CT285 t285 0 0.1f
M647 t282 nw40 t285 0 nch w=1u l=180n
M648 t285 t281 0 0 nch w=1u l=180n
M649 t283 nd9 vdd vdd pch w=2u l=180n
M650 t283 t281 vdd vdd pch w=2u l=180n
CT286 t286 0 0.1f
M651 t283 nd9 t286 0 nch w=1u l=180n
M652 t286 t281 0 0 nch w=1u l=180n
M653 nw41 t282 vdd vdd pch w=2u l=180n
M654 nw41 t283 vdd vdd pch w=2u l=180n
CT287 t287 0 0.1f
M655 nw41 t282 t287 0 nch w=1u l=180n
M656 t287 t283 0 0 nch w=1u l=180n
Cnw41 nw41 0 2f
CT288 t288 0 0.1f
CT289 t289 0 0.1f
CT290 t290 0 0.1f
M657 t288 nw41 vdd vdd pch w=2u l=180n
M658 t288 nd10 vdd vdd pch w=2u l=180n
CT291 t291 0 0.1f
M659 t288 nw41 t291 0 nch w=1u l=180n
M660 t291 nd10 0 0 nch w=1u l=180n
M661 t289 nw41 vdd vdd pch w=2u l=180n
M662 t289 t288 vdd vdd pch w=2u l=180n
CT292 t292 0 0.1f
M663 t289 nw41 t292 0 nch w=1u l=180n
M664 t292 t288 0 0 nch w=1u l=180n
M665 t290 nd10 vdd vdd pch w=2u l=180n
M666 t290 t288 vdd vdd pch w=2u l=180n
CT293 t293 0 0.1f
M667 t290 nd10 t293 0 nch w=1u l=180n
M668 t293 t288 0 0 nch w=1u l=180n
M669 nw42 t289 vdd vdd pch w=2u l=180n
M670 nw42 t290 vdd vdd pch w=2u l=180n
CT294 t294 0 0.1f
M671 nw42 t289 t294 0 nch w=1u l=180n
M672 t294 t290 0 0 nch w=1u l=180n
Cnw42 nw42 0 2f
CT295 t295 0 0.1f
CT296 t296 0 0.1f
CT297 t297 0 0.1f
M673 t295 nw42 vdd vdd pch w=2u l=180n
M674 t295 nd14 vdd vdd pch w=2u l=180n
CT298 t298 0 0.1f
M675 t295 nw42 t298 0 nch w=1u l=180n
M676 t298 nd14 0 0 nch w=1u l=180n
M677 t296 nw42 vdd vdd pch w=2u l=180n
M678 t296 t295 vdd vdd pch w=2u l=180n
CT299 t299 0 0.1f
M679 t296 nw42 t299 0 nch w=1u l=180n
M680 t299 t295 0 0 nch w=1u l=180n
M681 t297 nd14 vdd vdd pch w=2u l=180n
M682 t297 t295 vdd vdd pch w=2u l=180n
CT300 t300 0 0.1f
M683 t297 nd14 t300 0 nch w=1u l=180n
M684 t300 t295 0 0 nch w=1u l=180n
M685 nw43 t296 vdd vdd pch w=2u l=180n
M686 nw43 t297 vdd vdd pch w=2u l=180n
CT301 t301 0 0.1f
M687 nw43 t296 t301 0 nch w=1u l=180n
M688 t301 t297 0 0 nch w=1u l=180n
Cnw43 nw43 0 2f
CT302 t302 0 0.1f
CT303 t303 0 0.1f
CT304 t304 0 0.1f
M689 t302 nw43 vdd vdd pch w=2u l=180n
M690 t302 nd15 vdd vdd pch w=2u l=180n
CT305 t305 0 0.1f
M691 t302 nw43 t305 0 nch w=1u l=180n
M692 t305 nd15 0 0 nch w=1u l=180n
M693 t303 nw43 vdd vdd pch w=2u l=180n
M694 t303 t302 vdd vdd pch w=2u l=180n
CT306 t306 0 0.1f
M695 t303 nw43 t306 0 nch w=1u l=180n
M696 t306 t302 0 0 nch w=1u l=180n
M697 t304 nd15 vdd vdd pch w=2u l=180n
M698 t304 t302 vdd vdd pch w=2u l=180n
CT307 t307 0 0.1f
M699 t304 nd15 t307 0 nch w=1u l=180n
M700 t307 t302 0 0 nch w=1u l=180n
M701 nw44 t303 vdd vdd pch w=2u l=180n
M702 nw44 t304 vdd vdd pch w=2u l=180n
CT308 t308 0 0.1f
M703 nw44 t303 t308 0 nch w=1u l=180n
M704 t308 t304 0 0 nch w=1u l=180n
Cnw44 nw44 0 2f
CT309 t309 0 0.1f
CT310 t310 0 0.1f
CT311 t311 0 0.1f
M705 t309 nw44 vdd vdd pch w=2u l=180n
M706 t309 nd16 vdd vdd pch w=2u l=180n
CT312 t312 0 0.1f
M707 t309 nw44 t312 0 nch w=1u l=180n
M708 t312 nd16 0 0 nch w=1u l=180n
M709 t310 nw44 vdd vdd pch w=2u l=180n
M710 t310 t309 vdd vdd pch w=2u l=180n
CT313 t313 0 0.1f
M711 t310 nw44 t313 0 nch w=1u l=180n
M712 t313 t309 0 0 nch w=1u l=180n
M713 t311 nd16 vdd vdd pch w=2u l=180n
M714 t311 t309 vdd vdd pch w=2u l=180n
CT314 t314 0 0.1f
M715 t311 nd16 t314 0 nch w=1u l=180n
M716 t314 t309 0 0 nch w=1u l=180n
M717 nw45 t310 vdd vdd pch w=2u l=180n
M718 nw45 t311 vdd vdd pch w=2u l=180n
CT315 t315 0 0.1f
M719 nw45 t310 t315 0 nch w=1u l=180n
M720 t315 t311 0 0 nch w=1u l=180n
Cnw45 nw45 0 2f
CT316 t316 0 0.1f
CT317 t317 0 0.1f
CT318 t318 0 0.1f
M721 t316 nw45 vdd vdd pch w=2u l=180n
M722 t316 nd17 vdd vdd pch w=2u l=180n
CT319 t319 0 0.1f
M723 t316 nw45 t319 0 nch w=1u l=180n
M724 t319 nd17 0 0 nch w=1u l=180n
M725 t317 nw45 vdd vdd pch w=2u l=180n
M726 t317 t316 vdd vdd pch w=2u l=180n
CT320 t320 0 0.1f
M727 t317 nw45 t320 0 nch w=1u l=180n
M728 t320 t316 0 0 nch w=1u l=180n
M729 t318 nd17 vdd vdd pch w=2u l=180n
M730 t318 t316 vdd vdd pch w=2u l=180n
CT321 t321 0 0.1f
M731 t318 nd17 t321 0 nch w=1u l=180n
M732 t321 t316 0 0 nch w=1u l=180n
M733 nw46 t317 vdd vdd pch w=2u l=180n
M734 nw46 t318 vdd vdd pch w=2u l=180n
CT322 t322 0 0.1f
M735 nw46 t317 t322 0 nch w=1u l=180n
M736 t322 t318 0 0 nch w=1u l=180n
Cnw46 nw46 0 2f
CT323 t323 0 0.1f
CT324 t324 0 0.1f
CT325 t325 0 0.1f
M737 t323 nw46 vdd vdd pch w=2u l=180n
M738 t323 nd22 vdd vdd pch w=2u l=180n
CT326 t326 0 0.1f
M739 t323 nw46 t326 0 nch w=1u l=180n
M740 t326 nd22 0 0 nch w=1u l=180n
M741 t324 nw46 vdd vdd pch w=2u l=180n
M742 t324 t323 vdd vdd pch w=2u l=180n
CT327 t327 0 0.1f
M743 t324 nw46 t327 0 nch w=1u l=180n
M744 t327 t323 0 0 nch w=1u l=180n
M745 t325 nd22 vdd vdd pch w=2u l=180n
M746 t325 t323 vdd vdd pch w=2u l=180n
CT328 t328 0 0.1f
M747 t325 nd22 t328 0 nch w=1u l=180n
M748 t328 t323 0 0 nch w=1u l=180n
M749 nw47 t324 vdd vdd pch w=2u l=180n
M750 nw47 t325 vdd vdd pch w=2u l=180n
CT329 t329 0 0.1f
M751 nw47 t324 t329 0 nch w=1u l=180n
M752 t329 t325 0 0 nch w=1u l=180n
Cnw47 nw47 0 2f
CT330 t330 0 0.1f
CT331 t331 0 0.1f
CT332 t332 0 0.1f
M753 t330 nw47 vdd vdd pch w=2u l=180n
M754 t330 nd23 vdd vdd pch w=2u l=180n
CT333 t333 0 0.1f
M755 t330 nw47 t333 0 nch w=1u l=180n
M756 t333 nd23 0 0 nch w=1u l=180n
M757 t331 nw47 vdd vdd pch w=2u l=180n
M758 t331 t330 vdd vdd pch w=2u l=180n
CT334 t334 0 0.1f
M759 t331 nw47 t334 0 nch w=1u l=180n
M760 t334 t330 0 0 nch w=1u l=180n
M761 t332 nd23 vdd vdd pch w=2u l=180n
M762 t332 t330 vdd vdd pch w=2u l=180n
CT335 t335 0 0.1f
M763 t332 nd23 t335 0 nch w=1u l=180n
M764 t335 t330 0 0 nch w=1u l=180n
M765 nw48 t331 vdd vdd pch w=2u l=180n
M766 nw48 t332 vdd vdd pch w=2u l=180n
CT336 t336 0 0.1f
M767 nw48 t331 t336 0 nch w=1u l=180n
M768 t336 t332 0 0 nch w=1u l=180n
Cnw48 nw48 0 2f
CT337 t337 0 0.1f
CT338 t338 0 0.1f
CT339 t339 0 0.1f
M769 t337 nw48 vdd vdd pch w=2u l=180n
M770 t337 nd24 vdd vdd pch w=2u l=180n
CT340 t340 0 0.1f
M771 t337 nw48 t340 0 nch w=1u l=180n
M772 t340 nd24 0 0 nch w=1u l=180n
M773 t338 nw48 vdd vdd pch w=2u l=180n
M774 t338 t337 vdd vdd pch w=2u l=180n
CT341 t341 0 0.1f
M775 t338 nw48 t341 0 nch w=1u l=180n
M776 t341 t337 0 0 nch w=1u l=180n
M777 t339 nd24 vdd vdd pch w=2u l=180n
M778 t339 t337 vdd vdd pch w=2u l=180n
CT342 t342 0 0.1f
M779 t339 nd24 t342 0 nch w=1u l=180n
M780 t342 t337 0 0 nch w=1u l=180n
M781 nw49 t338 vdd vdd pch w=2u l=180n
M782 nw49 t339 vdd vdd pch w=2u l=180n
CT343 t343 0 0.1f
M783 nw49 t338 t343 0 nch w=1u l=180n
M784 t343 t339 0 0 nch w=1u l=180n
Cnw49 nw49 0 2f
CT344 t344 0 0.1f
CT345 t345 0 0.1f
CT346 t346 0 0.1f
M785 t344 nw49 vdd vdd pch w=2u l=180n
M786 t344 nd25 vdd vdd pch w=2u l=180n
CT347 t347 0 0.1f
M787 t344 nw49 t347 0 nch w=1u l=180n
M788 t347 nd25 0 0 nch w=1u l=180n
M789 t345 nw49 vdd vdd pch w=2u l=180n
M790 t345 t344 vdd vdd pch w=2u l=180n
CT348 t348 0 0.1f
M791 t345 nw49 t348 0 nch w=1u l=180n
M792 t348 t344 0 0 nch w=1u l=180n
M793 t346 nd25 vdd vdd pch w=2u l=180n
M794 t346 t344 vdd vdd pch w=2u l=180n
CT349 t349 0 0.1f
M795 t346 nd25 t349 0 nch w=1u l=180n
M796 t349 t344 0 0 nch w=1u l=180n
M797 nw50 t345 vdd vdd pch w=2u l=180n
M798 nw50 t346 vdd vdd pch w=2u l=180n
CT350 t350 0 0.1f
M799 nw50 t345 t350 0 nch w=1u l=180n
M800 t350 t346 0 0 nch w=1u l=180n
Cnw50 nw50 0 2f
CT351 t351 0 0.1f
CT352 t352 0 0.1f
CT353 t353 0 0.1f
M801 t351 nw50 vdd vdd pch w=2u l=180n
M802 t351 nd29 vdd vdd pch w=2u l=180n
CT354 t354 0 0.1f
M803 t351 nw50 t354 0 nch w=1u l=180n
M804 t354 nd29 0 0 nch w=1u l=180n
M805 t352 nw50 vdd vdd pch w=2u l=180n
M806 t352 t351 vdd vdd pch w=2u l=180n
CT355 t355 0 0.1f
M807 t352 nw50 t355 0 nch w=1u l=180n
M808 t355 t351 0 0 nch w=1u l=180n
M809 t353 nd29 vdd vdd pch w=2u l=180n
M810 t353 t351 vdd vdd pch w=2u l=180n
CT356 t356 0 0.1f
M811 t353 nd29 t356 0 nch w=1u l=180n
M812 t356 t351 0 0 nch w=1u l=180n
M813 nw51 t352 vdd vdd pch w=2u l=180n
M814 nw51 t353 vdd vdd pch w=2u l=180n
CT357 t357 0 0.1f
M815 nw51 t352 t357 0 nch w=1u l=180n
M816 t357 t353 0 0 nch w=1u l=180n
Cnw51 nw51 0 2f
CT358 t358 0 0.1f
CT359 t359 0 0.1f
CT360 t360 0 0.1f
M817 t358 nw51 vdd vdd pch w=2u l=180n
M818 t358 nd30 vdd vdd pch w=2u l=180n
CT361 t361 0 0.1f
M819 t358 nw51 t361 0 nch w=1u l=180n
M820 t361 nd30 0 0 nch w=1u l=180n
M821 t359 nw51 vdd vdd pch w=2u l=180n
M822 t359 t358 vdd vdd pch w=2u l=180n
CT362 t362 0 0.1f
M823 t359 nw51 t362 0 nch w=1u l=180n
M824 t362 t358 0 0 nch w=1u l=180n
M825 t360 nd30 vdd vdd pch w=2u l=180n
M826 t360 t358 vdd vdd pch w=2u l=180n
CT363 t363 0 0.1f
M827 t360 nd30 t363 0 nch w=1u l=180n
M828 t363 t358 0 0 nch w=1u l=180n
M829 nw52 t359 vdd vdd pch w=2u l=180n
M830 nw52 t360 vdd vdd pch w=2u l=180n
CT364 t364 0 0.1f
M831 nw52 t359 t364 0 nch w=1u l=180n
M832 t364 t360 0 0 nch w=1u l=180n
Cnw52 nw52 0 2f
CT365 t365 0 0.1f
CT366 t366 0 0.1f
CT367 t367 0 0.1f
M833 t365 nw52 vdd vdd pch w=2u l=180n
M834 t365 nd31 vdd vdd pch w=2u l=180n
CT368 t368 0 0.1f
M835 t365 nw52 t368 0 nch w=1u l=180n
M836 t368 nd31 0 0 nch w=1u l=180n
M837 t366 nw52 vdd vdd pch w=2u l=180n
M838 t366 t365 vdd vdd pch w=2u l=180n
CT369 t369 0 0.1f
M839 t366 nw52 t369 0 nch w=1u l=180n
M840 t369 t365 0 0 nch w=1u l=180n
M841 t367 nd31 vdd vdd pch w=2u l=180n
M842 t367 t365 vdd vdd pch w=2u l=180n
CT370 t370 0 0.1f
M843 t367 nd31 t370 0 nch w=1u l=180n
M844 t370 t365 0 0 nch w=1u l=180n
M845 nw53 t366 vdd vdd pch w=2u l=180n
M846 nw53 t367 vdd vdd pch w=2u l=180n
CT371 t371 0 0.1f
M847 nw53 t366 t371 0 nch w=1u l=180n
M848 t371 t367 0 0 nch w=1u l=180n
Cnw53 nw53 0 2f
CT372 t372 0 0.1f
CT373 t373 0 0.1f
CT374 t374 0 0.1f
M849 t372 nw53 vdd vdd pch w=2u l=180n
M850 t372 nr2 vdd vdd pch w=2u l=180n
CT375 t375 0 0.1f
M851 t372 nw53 t375 0 nch w=1u l=180n
M852 t375 nr2 0 0 nch w=1u l=180n
M853 t373 nw53 vdd vdd pch w=2u l=180n
M854 t373 t372 vdd vdd pch w=2u l=180n
CT376 t376 0 0.1f
M855 t373 nw53 t376 0 nch w=1u l=180n
M856 t376 t372 0 0 nch w=1u l=180n
M857 t374 nr2 vdd vdd pch w=2u l=180n
M858 t374 t372 vdd vdd pch w=2u l=180n
CT377 t377 0 0.1f
M859 t374 nr2 t377 0 nch w=1u l=180n
M860 t377 t372 0 0 nch w=1u l=180n
M861 nw54 t373 vdd vdd pch w=2u l=180n
M862 nw54 t374 vdd vdd pch w=2u l=180n
CT378 t378 0 0.1f
M863 nw54 t373 t378 0 nch w=1u l=180n
M864 t378 t374 0 0 nch w=1u l=180n
Cnw54 nw54 0 2f
CT379 t379 0 0.1f
CT380 t380 0 0.1f
CT381 t381 0 0.1f
M865 t379 nd4 vdd vdd pch w=2u l=180n
M866 t379 nd5 vdd vdd pch w=2u l=180n
CT382 t382 0 0.1f
M867 t379 nd4 t382 0 nch w=1u l=180n
M868 t382 nd5 0 0 nch w=1u l=180n
M869 t380 nd4 vdd vdd pch w=2u l=180n
M870 t380 t379 vdd vdd pch w=2u l=180n
CT383 t383 0 0.1f
M871 t380 nd4 t383 0 nch w=1u l=180n
M872 t383 t379 0 0 nch w=1u l=180n
M873 t381 nd5 vdd vdd pch w=2u l=180n
M874 t381 t379 vdd vdd pch w=2u l=180n
CT384 t384 0 0.1f
M875 t381 nd5 t384 0 nch w=1u l=180n
M876 t384 t379 0 0 nch w=1u l=180n
M877 nw55 t380 vdd vdd pch w=2u l=180n
M878 nw55 t381 vdd vdd pch w=2u l=180n
CT385 t385 0 0.1f
M879 nw55 t380 t385 0 nch w=1u l=180n
M880 t385 t381 0 0 nch w=1u l=180n
Cnw55 nw55 0 2f
CT386 t386 0 0.1f
CT387 t387 0 0.1f
CT388 t388 0 0.1f
M881 t386 nw55 vdd vdd pch w=2u l=180n
M882 t386 nd6 vdd vdd pch w=2u l=180n
CT389 t389 0 0.1f
M883 t386 nw55 t389 0 nch w=1u l=180n
M884 t389 nd6 0 0 nch w=1u l=180n
M885 t387 nw55 vdd vdd pch w=2u l=180n
M886 t387 t386 vdd vdd pch w=2u l=180n
CT390 t390 0 0.1f
M887 t387 nw55 t390 0 nch w=1u l=180n
M888 t390 t386 0 0 nch w=1u l=180n
M889 t388 nd6 vdd vdd pch w=2u l=180n
M890 t388 t386 vdd vdd pch w=2u l=180n
CT391 t391 0 0.1f
M891 t388 nd6 t391 0 nch w=1u l=180n
M892 t391 t386 0 0 nch w=1u l=180n
M893 nw56 t387 vdd vdd pch w=2u l=180n
M894 nw56 t388 vdd vdd pch w=2u l=180n
CT392 t392 0 0.1f
M895 nw56 t387 t392 0 nch w=1u l=180n
M896 t392 t388 0 0 nch w=1u l=180n
Cnw56 nw56 0 2f
CT393 t393 0 0.1f
CT394 t394 0 0.1f
CT395 t395 0 0.1f
M897 t393 nw56 vdd vdd pch w=2u l=180n
M898 t393 nd7 vdd vdd pch w=2u l=180n
CT396 t396 0 0.1f
M899 t393 nw56 t396 0 nch w=1u l=180n
M900 t396 nd7 0 0 nch w=1u l=180n
M901 t394 nw56 vdd vdd pch w=2u l=180n
M902 t394 t393 vdd vdd pch w=2u l=180n
CT397 t397 0 0.1f
M903 t394 nw56 t397 0 nch w=1u l=180n
M904 t397 t393 0 0 nch w=1u l=180n
M905 t395 nd7 vdd vdd pch w=2u l=180n
M906 t395 t393 vdd vdd pch w=2u l=180n
CT398 t398 0 0.1f
M907 t395 nd7 t398 0 nch w=1u l=180n
M908 t398 t393 0 0 nch w=1u l=180n
M909 nw57 t394 vdd vdd pch w=2u l=180n
M910 nw57 t395 vdd vdd pch w=2u l=180n
CT399 t399 0 0.1f
M911 nw57 t394 t399 0 nch w=1u l=180n
M912 t399 t395 0 0 nch w=1u l=180n
Cnw57 nw57 0 2f
CT400 t400 0 0.1f
CT401 t401 0 0.1f
CT402 t402 0 0.1f
M913 t400 nw57 vdd vdd pch w=2u l=180n
M914 t400 nd8 vdd vdd pch w=2u l=180n
CT403 t403 0 0.1f
M915 t400 nw57 t403 0 nch w=1u l=180n
M916 t403 nd8 0 0 nch w=1u l=180n
M917 t401 nw57 vdd vdd pch w=2u l=180n
M918 t401 t400 vdd vdd pch w=2u l=180n
CT404 t404 0 0.1f
M919 t401 nw57 t404 0 nch w=1u l=180n
M920 t404 t400 0 0 nch w=1u l=180n
M921 t402 nd8 vdd vdd pch w=2u l=180n
M922 t402 t400 vdd vdd pch w=2u l=180n
CT405 t405 0 0.1f
M923 t402 nd8 t405 0 nch w=1u l=180n
M924 t405 t400 0 0 nch w=1u l=180n
M925 nw58 t401 vdd vdd pch w=2u l=180n
M926 nw58 t402 vdd vdd pch w=2u l=180n
CT406 t406 0 0.1f
M927 nw58 t401 t406 0 nch w=1u l=180n
M928 t406 t402 0 0 nch w=1u l=180n
Cnw58 nw58 0 2f
CT407 t407 0 0.1f
CT408 t408 0 0.1f
CT409 t409 0 0.1f
M929 t407 nw58 vdd vdd pch w=2u l=180n
M930 t407 nd9 vdd vdd pch w=2u l=180n
CT410 t410 0 0.1f
M931 t407 nw58 t410 0 nch w=1u l=180n
M932 t410 nd9 0 0 nch w=1u l=180n
M933 t408 nw58 vdd vdd pch w=2u l=180n
M934 t408 t407 vdd vdd pch w=2u l=180n
CT411 t411 0 0.1f
M935 t408 nw58 t411 0 nch w=1u l=180n
M936 t411 t407 0 0 nch w=1u l=180n
M937 t409 nd9 vdd vdd pch w=2u l=180n
M938 t409 t407 vdd vdd pch w=2u l=180n
CT412 t412 0 0.1f
M939 t409 nd9 t412 0 nch w=1u l=180n
M940 t412 t407 0 0 nch w=1u l=180n
M941 nw59 t408 vdd vdd pch w=2u l=180n
M942 nw59 t409 vdd vdd pch w=2u l=180n
CT413 t413 0 0.1f
M943 nw59 t408 t413 0 nch w=1u l=180n
M944 t413 t409 0 0 nch w=1u l=180n
Cnw59 nw59 0 2f
CT414 t414 0 0.1f
CT415 t415 0 0.1f
CT416 t416 0 0.1f
M945 t414 nw59 vdd vdd pch w=2u l=180n
M946 t414 nd10 vdd vdd pch w=2u l=180n
CT417 t417 0 0.1f
M947 t414 nw59 t417 0 nch w=1u l=180n
M948 t417 nd10 0 0 nch w=1u l=180n
M949 t415 nw59 vdd vdd pch w=2u l=180n
M950 t415 t414 vdd vdd pch w=2u l=180n
CT418 t418 0 0.1f
M951 t415 nw59 t418 0 nch w=1u l=180n
M952 t418 t414 0 0 nch w=1u l=180n
M953 t416 nd10 vdd vdd pch w=2u l=180n
M954 t416 t414 vdd vdd pch w=2u l=180n
CT419 t419 0 0.1f
M955 t416 nd10 t419 0 nch w=1u l=180n
M956 t419 t414 0 0 nch w=1u l=180n
M957 nw60 t415 vdd vdd pch w=2u l=180n
M958 nw60 t416 vdd vdd pch w=2u l=180n
CT420 t420 0 0.1f
M959 nw60 t415 t420 0 nch w=1u l=180n
M960 t420 t416 0 0 nch w=1u l=180n
Cnw60 nw60 0 2f
CT421 t421 0 0.1f
CT422 t422 0 0.1f
CT423 t423 0 0.1f
M961 t421 nw60 vdd vdd pch w=2u l=180n
M962 t421 nd18 vdd vdd pch w=2u l=180n
CT424 t424 0 0.1f
M963 t421 nw60 t424 0 nch w=1u l=180n
M964 t424 nd18 0 0 nch w=1u l=180n
M965 t422 nw60 vdd vdd pch w=2u l=180n
M966 t422 t421 vdd vdd pch w=2u l=180n
CT425 t425 0 0.1f
M967 t422 nw60 t425 0 nch w=1u l=180n
M968 t425 t421 0 0 nch w=1u l=180n
M969 t423 nd18 vdd vdd pch w=2u l=180n
M970 t423 t421 vdd vdd pch w=2u l=180n
CT426 t426 0 0.1f
M971 t423 nd18 t426 0 nch w=1u l=180n
M972 t426 t421 0 0 nch w=1u l=180n
M973 nw61 t422 vdd vdd pch w=2u l=180n
M974 nw61 t423 vdd vdd pch w=2u l=180n
CT427 t427 0 0.1f
M975 nw61 t422 t427 0 nch w=1u l=180n
M976 t427 t423 0 0 nch w=1u l=180n
Cnw61 nw61 0 2f
CT428 t428 0 0.1f
CT429 t429 0 0.1f
CT430 t430 0 0.1f
M977 t428 nw61 vdd vdd pch w=2u l=180n
M978 t428 nd19 vdd vdd pch w=2u l=180n
CT431 t431 0 0.1f
M979 t428 nw61 t431 0 nch w=1u l=180n
M980 t431 nd19 0 0 nch w=1u l=180n
M981 t429 nw61 vdd vdd pch w=2u l=180n
M982 t429 t428 vdd vdd pch w=2u l=180n
CT432 t432 0 0.1f
M983 t429 nw61 t432 0 nch w=1u l=180n
M984 t432 t428 0 0 nch w=1u l=180n
M985 t430 nd19 vdd vdd pch w=2u l=180n
M986 t430 t428 vdd vdd pch w=2u l=180n
CT433 t433 0 0.1f
M987 t430 nd19 t433 0 nch w=1u l=180n
M988 t433 t428 0 0 nch w=1u l=180n
M989 nw62 t429 vdd vdd pch w=2u l=180n
M990 nw62 t430 vdd vdd pch w=2u l=180n
CT434 t434 0 0.1f
M991 nw62 t429 t434 0 nch w=1u l=180n
M992 t434 t430 0 0 nch w=1u l=180n
Cnw62 nw62 0 2f
CT435 t435 0 0.1f
CT436 t436 0 0.1f
CT437 t437 0 0.1f
M993 t435 nw62 vdd vdd pch w=2u l=180n
M994 t435 nd20 vdd vdd pch w=2u l=180n
CT438 t438 0 0.1f
M995 t435 nw62 t438 0 nch w=1u l=180n
M996 t438 nd20 0 0 nch w=1u l=180n
M997 t436 nw62 vdd vdd pch w=2u l=180n
M998 t436 t435 vdd vdd pch w=2u l=180n
CT439 t439 0 0.1f
M999 t436 nw62 t439 0 nch w=1u l=180n
M1000 t439 t435 0 0 nch w=1u l=180n
M1001 t437 nd20 vdd vdd pch w=2u l=180n
M1002 t437 t435 vdd vdd pch w=2u l=180n
CT440 t440 0 0.1f
M1003 t437 nd20 t440 0 nch w=1u l=180n
M1004 t440 t435 0 0 nch w=1u l=180n
M1005 nw63 t436 vdd vdd pch w=2u l=180n
M1006 nw63 t437 vdd vdd pch w=2u l=180n
CT441 t441 0 0.1f
M1007 nw63 t436 t441 0 nch w=1u l=180n
M1008 t441 t437 0 0 nch w=1u l=180n
Cnw63 nw63 0 2f
CT442 t442 0 0.1f
CT443 t443 0 0.1f
CT444 t444 0 0.1f
M1009 t442 nw63 vdd vdd pch w=2u l=180n
M1010 t442 nd21 vdd vdd pch w=2u l=180n
CT445 t445 0 0.1f
M1011 t442 nw63 t445 0 nch w=1u l=180n
M1012 t445 nd21 0 0 nch w=1u l=180n
M1013 t443 nw63 vdd vdd pch w=2u l=180n
M1014 t443 t442 vdd vdd pch w=2u l=180n
CT446 t446 0 0.1f
M1015 t443 nw63 t446 0 nch w=1u l=180n
M1016 t446 t442 0 0 nch w=1u l=180n
M1017 t444 nd21 vdd vdd pch w=2u l=180n
M1018 t444 t442 vdd vdd pch w=2u l=180n
CT447 t447 0 0.1f
M1019 t444 nd21 t447 0 nch w=1u l=180n
M1020 t447 t442 0 0 nch w=1u l=180n
M1021 nw64 t443 vdd vdd pch w=2u l=180n
M1022 nw64 t444 vdd vdd pch w=2u l=180n
CT448 t448 0 0.1f
M1023 nw64 t443 t448 0 nch w=1u l=180n
M1024 t448 t444 0 0 nch w=1u l=180n
Cnw64 nw64 0 2f
CT449 t449 0 0.1f
CT450 t450 0 0.1f
CT451 t451 0 0.1f
M1025 t449 nw64 vdd vdd pch w=2u l=180n
M1026 t449 nd22 vdd vdd pch w=2u l=180n
CT452 t452 0 0.1f
M1027 t449 nw64 t452 0 nch w=1u l=180n
M1028 t452 nd22 0 0 nch w=1u l=180n
M1029 t450 nw64 vdd vdd pch w=2u l=180n
M1030 t450 t449 vdd vdd pch w=2u l=180n
CT453 t453 0 0.1f
M1031 t450 nw64 t453 0 nch w=1u l=180n
M1032 t453 t449 0 0 nch w=1u l=180n
M1033 t451 nd22 vdd vdd pch w=2u l=180n
M1034 t451 t449 vdd vdd pch w=2u l=180n
CT454 t454 0 0.1f
M1035 t451 nd22 t454 0 nch w=1u l=180n
M1036 t454 t449 0 0 nch w=1u l=180n
M1037 nw65 t450 vdd vdd pch w=2u l=180n
M1038 nw65 t451 vdd vdd pch w=2u l=180n
CT455 t455 0 0.1f
M1039 nw65 t450 t455 0 nch w=1u l=180n
M1040 t455 t451 0 0 nch w=1u l=180n
Cnw65 nw65 0 2f
CT456 t456 0 0.1f
CT457 t457 0 0.1f
CT458 t458 0 0.1f
M1041 t456 nw65 vdd vdd pch w=2u l=180n
M1042 t456 nd23 vdd vdd pch w=2u l=180n
CT459 t459 0 0.1f
M1043 t456 nw65 t459 0 nch w=1u l=180n
M1044 t459 nd23 0 0 nch w=1u l=180n
M1045 t457 nw65 vdd vdd pch w=2u l=180n
M1046 t457 t456 vdd vdd pch w=2u l=180n
CT460 t460 0 0.1f
M1047 t457 nw65 t460 0 nch w=1u l=180n
M1048 t460 t456 0 0 nch w=1u l=180n
M1049 t458 nd23 vdd vdd pch w=2u l=180n
M1050 t458 t456 vdd vdd pch w=2u l=180n
CT461 t461 0 0.1f
M1051 t458 nd23 t461 0 nch w=1u l=180n
M1052 t461 t456 0 0 nch w=1u l=180n
M1053 nw66 t457 vdd vdd pch w=2u l=180n
M1054 nw66 t458 vdd vdd pch w=2u l=180n
CT462 t462 0 0.1f
M1055 nw66 t457 t462 0 nch w=1u l=180n
M1056 t462 t458 0 0 nch w=1u l=180n
Cnw66 nw66 0 2f
CT463 t463 0 0.1f
CT464 t464 0 0.1f
CT465 t465 0 0.1f
M1057 t463 nw66 vdd vdd pch w=2u l=180n
M1058 t463 nd24 vdd vdd pch w=2u l=180n
CT466 t466 0 0.1f
M1059 t463 nw66 t466 0 nch w=1u l=180n
M1060 t466 nd24 0 0 nch w=1u l=180n
M1061 t464 nw66 vdd vdd pch w=2u l=180n
M1062 t464 t463 vdd vdd pch w=2u l=180n
CT467 t467 0 0.1f
M1063 t464 nw66 t467 0 nch w=1u l=180n
M1064 t467 t463 0 0 nch w=1u l=180n
M1065 t465 nd24 vdd vdd pch w=2u l=180n
M1066 t465 t463 vdd vdd pch w=2u l=180n
CT468 t468 0 0.1f
M1067 t465 nd24 t468 0 nch w=1u l=180n
M1068 t468 t463 0 0 nch w=1u l=180n
M1069 nw67 t464 vdd vdd pch w=2u l=180n
M1070 nw67 t465 vdd vdd pch w=2u l=180n
CT469 t469 0 0.1f
M1071 nw67 t464 t469 0 nch w=1u l=180n
M1072 t469 t465 0 0 nch w=1u l=180n
Cnw67 nw67 0 2f
CT470 t470 0 0.1f
CT471 t471 0 0.1f
CT472 t472 0 0.1f
M1073 t470 nw67 vdd vdd pch w=2u l=180n
M1074 t470 nd25 vdd vdd pch w=2u l=180n
CT473 t473 0 0.1f
M1075 t470 nw67 t473 0 nch w=1u l=180n
M1076 t473 nd25 0 0 nch w=1u l=180n
M1077 t471 nw67 vdd vdd pch w=2u l=180n
M1078 t471 t470 vdd vdd pch w=2u l=180n
CT474 t474 0 0.1f
M1079 t471 nw67 t474 0 nch w=1u l=180n
M1080 t474 t470 0 0 nch w=1u l=180n
M1081 t472 nd25 vdd vdd pch w=2u l=180n
M1082 t472 t470 vdd vdd pch w=2u l=180n
CT475 t475 0 0.1f
M1083 t472 nd25 t475 0 nch w=1u l=180n
M1084 t475 t470 0 0 nch w=1u l=180n
M1085 nw68 t471 vdd vdd pch w=2u l=180n
M1086 nw68 t472 vdd vdd pch w=2u l=180n
CT476 t476 0 0.1f
M1087 nw68 t471 t476 0 nch w=1u l=180n
M1088 t476 t472 0 0 nch w=1u l=180n
Cnw68 nw68 0 2f
CT477 t477 0 0.1f
CT478 t478 0 0.1f
CT479 t479 0 0.1f
M1089 t477 nw68 vdd vdd pch w=2u l=180n
M1090 t477 nr3 vdd vdd pch w=2u l=180n
CT480 t480 0 0.1f
M1091 t477 nw68 t480 0 nch w=1u l=180n
M1092 t480 nr3 0 0 nch w=1u l=180n
M1093 t478 nw68 vdd vdd pch w=2u l=180n
M1094 t478 t477 vdd vdd pch w=2u l=180n
CT481 t481 0 0.1f
M1095 t478 nw68 t481 0 nch w=1u l=180n
M1096 t481 t477 0 0 nch w=1u l=180n
M1097 t479 nr3 vdd vdd pch w=2u l=180n
M1098 t479 t477 vdd vdd pch w=2u l=180n
CT482 t482 0 0.1f
M1099 t479 nr3 t482 0 nch w=1u l=180n
M1100 t482 t477 0 0 nch w=1u l=180n
M1101 nw69 t478 vdd vdd pch w=2u l=180n
M1102 nw69 t479 vdd vdd pch w=2u l=180n
CT483 t483 0 0.1f
M1103 nw69 t478 t483 0 nch w=1u l=180n
M1104 t483 t479 0 0 nch w=1u l=180n
Cnw69 nw69 0 2f
CT484 t484 0 0.1f
CT485 t485 0 0.1f
CT486 t486 0 0.1f
M1105 t484 nd11 vdd vdd pch w=2u l=180n
M1106 t484 nd12 vdd vdd pch w=2u l=180n
CT487 t487 0 0.1f
M1107 t484 nd11 t487 0 nch w=1u l=180n
M1108 t487 nd12 0 0 nch w=1u l=180n
M1109 t485 nd11 vdd vdd pch w=2u l=180n
M1110 t485 t484 vdd vdd pch w=2u l=180n
CT488 t488 0 0.1f
M1111 t485 nd11 t488 0 nch w=1u l=180n
M1112 t488 t484 0 0 nch w=1u l=180n
M1113 t486 nd12 vdd vdd pch w=2u l=180n
M1114 t486 t484 vdd vdd pch w=2u l=180n
CT489 t489 0 0.1f
M1115 t486 nd12 t489 0 nch w=1u l=180n
M1116 t489 t484 0 0 nch w=1u l=180n
M1117 nw70 t485 vdd vdd pch w=2u l=180n
M1118 nw70 t486 vdd vdd pch w=2u l=180n
CT490 t490 0 0.1f
M1119 nw70 t485 t490 0 nch w=1u l=180n
M1120 t490 t486 0 0 nch w=1u l=180n
Cnw70 nw70 0 2f
CT491 t491 0 0.1f
CT492 t492 0 0.1f
CT493 t493 0 0.1f
M1121 t491 nw70 vdd vdd pch w=2u l=180n
M1122 t491 nd13 vdd vdd pch w=2u l=180n
CT494 t494 0 0.1f
M1123 t491 nw70 t494 0 nch w=1u l=180n
M1124 t494 nd13 0 0 nch w=1u l=180n
M1125 t492 nw70 vdd vdd pch w=2u l=180n
M1126 t492 t491 vdd vdd pch w=2u l=180n
CT495 t495 0 0.1f
M1127 t492 nw70 t495 0 nch w=1u l=180n
M1128 t495 t491 0 0 nch w=1u l=180n
M1129 t493 nd13 vdd vdd pch w=2u l=180n
M1130 t493 t491 vdd vdd pch w=2u l=180n
CT496 t496 0 0.1f
M1131 t493 nd13 t496 0 nch w=1u l=180n
M1132 t496 t491 0 0 nch w=1u l=180n
M1133 nw71 t492 vdd vdd pch w=2u l=180n
M1134 nw71 t493 vdd vdd pch w=2u l=180n
CT497 t497 0 0.1f
M1135 nw71 t492 t497 0 nch w=1u l=180n
M1136 t497 t493 0 0 nch w=1u l=180n
Cnw71 nw71 0 2f
CT498 t498 0 0.1f
CT499 t499 0 0.1f
CT500 t500 0 0.1f
M1137 t498 nw71 vdd vdd pch w=2u l=180n
M1138 t498 nd14 vdd vdd pch w=2u l=180n
CT501 t501 0 0.1f
M1139 t498 nw71 t501 0 nch w=1u l=180n
M1140 t501 nd14 0 0 nch w=1u l=180n
M1141 t499 nw71 vdd vdd pch w=2u l=180n
M1142 t499 t498 vdd vdd pch w=2u l=180n
CT502 t502 0 0.1f
M1143 t499 nw71 t502 0 nch w=1u l=180n
M1144 t502 t498 0 0 nch w=1u l=180n
M1145 t500 nd14 vdd vdd pch w=2u l=180n
M1146 t500 t498 vdd vdd pch w=2u l=180n
CT503 t503 0 0.1f
M1147 t500 nd14 t503 0 nch w=1u l=180n
M1148 t503 t498 0 0 nch w=1u l=180n
M1149 nw72 t499 vdd vdd pch w=2u l=180n
M1150 nw72 t500 vdd vdd pch w=2u l=180n
CT504 t504 0 0.1f
M1151 nw72 t499 t504 0 nch w=1u l=180n
M1152 t504 t500 0 0 nch w=1u l=180n
Cnw72 nw72 0 2f
CT505 t505 0 0.1f
CT506 t506 0 0.1f
CT507 t507 0 0.1f
M1153 t505 nw72 vdd vdd pch w=2u l=180n
M1154 t505 nd15 vdd vdd pch w=2u l=180n
CT508 t508 0 0.1f
M1155 t505 nw72 t508 0 nch w=1u l=180n
M1156 t508 nd15 0 0 nch w=1u l=180n
M1157 t506 nw72 vdd vdd pch w=2u l=180n
M1158 t506 t505 vdd vdd pch w=2u l=180n
CT509 t509 0 0.1f
M1159 t506 nw72 t509 0 nch w=1u l=180n
M1160 t509 t505 0 0 nch w=1u l=180n
M1161 t507 nd15 vdd vdd pch w=2u l=180n
M1162 t507 t505 vdd vdd pch w=2u l=180n
CT510 t510 0 0.1f
M1163 t507 nd15 t510 0 nch w=1u l=180n
M1164 t510 t505 0 0 nch w=1u l=180n
M1165 nw73 t506 vdd vdd pch w=2u l=180n
M1166 nw73 t507 vdd vdd pch w=2u l=180n
CT511 t511 0 0.1f
M1167 nw73 t506 t511 0 nch w=1u l=180n
M1168 t511 t507 0 0 nch w=1u l=180n
Cnw73 nw73 0 2f
CT512 t512 0 0.1f
CT513 t513 0 0.1f
CT514 t514 0 0.1f
M1169 t512 nw73 vdd vdd pch w=2u l=180n
M1170 t512 nd16 vdd vdd pch w=2u l=180n
CT515 t515 0 0.1f
M1171 t512 nw73 t515 0 nch w=1u l=180n
M1172 t515 nd16 0 0 nch w=1u l=180n
M1173 t513 nw73 vdd vdd pch w=2u l=180n
M1174 t513 t512 vdd vdd pch w=2u l=180n
CT516 t516 0 0.1f
M1175 t513 nw73 t516 0 nch w=1u l=180n
M1176 t516 t512 0 0 nch w=1u l=180n
M1177 t514 nd16 vdd vdd pch w=2u l=180n
M1178 t514 t512 vdd vdd pch w=2u l=180n
CT517 t517 0 0.1f
M1179 t514 nd16 t517 0 nch w=1u l=180n
M1180 t517 t512 0 0 nch w=1u l=180n
M1181 nw74 t513 vdd vdd pch w=2u l=180n
M1182 nw74 t514 vdd vdd pch w=2u l=180n
CT518 t518 0 0.1f
M1183 nw74 t513 t518 0 nch w=1u l=180n
M1184 t518 t514 0 0 nch w=1u l=180n
Cnw74 nw74 0 2f
CT519 t519 0 0.1f
CT520 t520 0 0.1f
CT521 t521 0 0.1f
M1185 t519 nw74 vdd vdd pch w=2u l=180n
M1186 t519 nd17 vdd vdd pch w=2u l=180n
CT522 t522 0 0.1f
M1187 t519 nw74 t522 0 nch w=1u l=180n
M1188 t522 nd17 0 0 nch w=1u l=180n
M1189 t520 nw74 vdd vdd pch w=2u l=180n
M1190 t520 t519 vdd vdd pch w=2u l=180n
CT523 t523 0 0.1f
M1191 t520 nw74 t523 0 nch w=1u l=180n
M1192 t523 t519 0 0 nch w=1u l=180n
M1193 t521 nd17 vdd vdd pch w=2u l=180n
M1194 t521 t519 vdd vdd pch w=2u l=180n
CT524 t524 0 0.1f
M1195 t521 nd17 t524 0 nch w=1u l=180n
M1196 t524 t519 0 0 nch w=1u l=180n
M1197 nw75 t520 vdd vdd pch w=2u l=180n
M1198 nw75 t521 vdd vdd pch w=2u l=180n
CT525 t525 0 0.1f
M1199 nw75 t520 t525 0 nch w=1u l=180n
M1200 t525 t521 0 0 nch w=1u l=180n
Cnw75 nw75 0 2f
CT526 t526 0 0.1f
CT527 t527 0 0.1f
CT528 t528 0 0.1f
M1201 t526 nw75 vdd vdd pch w=2u l=180n
M1202 t526 nd18 vdd vdd pch w=2u l=180n
CT529 t529 0 0.1f
M1203 t526 nw75 t529 0 nch w=1u l=180n
M1204 t529 nd18 0 0 nch w=1u l=180n
M1205 t527 nw75 vdd vdd pch w=2u l=180n
M1206 t527 t526 vdd vdd pch w=2u l=180n
CT530 t530 0 0.1f
M1207 t527 nw75 t530 0 nch w=1u l=180n
M1208 t530 t526 0 0 nch w=1u l=180n
M1209 t528 nd18 vdd vdd pch w=2u l=180n
M1210 t528 t526 vdd vdd pch w=2u l=180n
CT531 t531 0 0.1f
M1211 t528 nd18 t531 0 nch w=1u l=180n
M1212 t531 t526 0 0 nch w=1u l=180n
M1213 nw76 t527 vdd vdd pch w=2u l=180n
M1214 nw76 t528 vdd vdd pch w=2u l=180n
CT532 t532 0 0.1f
M1215 nw76 t527 t532 0 nch w=1u l=180n
M1216 t532 t528 0 0 nch w=1u l=180n
Cnw76 nw76 0 2f
CT533 t533 0 0.1f
CT534 t534 0 0.1f
CT535 t535 0 0.1f
M1217 t533 nw76 vdd vdd pch w=2u l=180n
M1218 t533 nd19 vdd vdd pch w=2u l=180n
CT536 t536 0 0.1f
M1219 t533 nw76 t536 0 nch w=1u l=180n
M1220 t536 nd19 0 0 nch w=1u l=180n
M1221 t534 nw76 vdd vdd pch w=2u l=180n
M1222 t534 t533 vdd vdd pch w=2u l=180n
CT537 t537 0 0.1f
M1223 t534 nw76 t537 0 nch w=1u l=180n
M1224 t537 t533 0 0 nch w=1u l=180n
M1225 t535 nd19 vdd vdd pch w=2u l=180n
M1226 t535 t533 vdd vdd pch w=2u l=180n
CT538 t538 0 0.1f
M1227 t535 nd19 t538 0 nch w=1u l=180n
M1228 t538 t533 0 0 nch w=1u l=180n
M1229 nw77 t534 vdd vdd pch w=2u l=180n
M1230 nw77 t535 vdd vdd pch w=2u l=180n
CT539 t539 0 0.1f
M1231 nw77 t534 t539 0 nch w=1u l=180n
M1232 t539 t535 0 0 nch w=1u l=180n
Cnw77 nw77 0 2f
CT540 t540 0 0.1f
CT541 t541 0 0.1f
CT542 t542 0 0.1f
M1233 t540 nw77 vdd vdd pch w=2u l=180n
M1234 t540 nd20 vdd vdd pch w=2u l=180n
CT543 t543 0 0.1f
M1235 t540 nw77 t543 0 nch w=1u l=180n
M1236 t543 nd20 0 0 nch w=1u l=180n
M1237 t541 nw77 vdd vdd pch w=2u l=180n
M1238 t541 t540 vdd vdd pch w=2u l=180n
CT544 t544 0 0.1f
M1239 t541 nw77 t544 0 nch w=1u l=180n
M1240 t544 t540 0 0 nch w=1u l=180n
M1241 t542 nd20 vdd vdd pch w=2u l=180n
M1242 t542 t540 vdd vdd pch w=2u l=180n
CT545 t545 0 0.1f
M1243 t542 nd20 t545 0 nch w=1u l=180n
M1244 t545 t540 0 0 nch w=1u l=180n
M1245 nw78 t541 vdd vdd pch w=2u l=180n
M1246 nw78 t542 vdd vdd pch w=2u l=180n
CT546 t546 0 0.1f
M1247 nw78 t541 t546 0 nch w=1u l=180n
M1248 t546 t542 0 0 nch w=1u l=180n
Cnw78 nw78 0 2f
CT547 t547 0 0.1f
CT548 t548 0 0.1f
CT549 t549 0 0.1f
M1249 t547 nw78 vdd vdd pch w=2u l=180n
M1250 t547 nd21 vdd vdd pch w=2u l=180n
CT550 t550 0 0.1f
M1251 t547 nw78 t550 0 nch w=1u l=180n
M1252 t550 nd21 0 0 nch w=1u l=180n
M1253 t548 nw78 vdd vdd pch w=2u l=180n
M1254 t548 t547 vdd vdd pch w=2u l=180n
CT551 t551 0 0.1f
M1255 t548 nw78 t551 0 nch w=1u l=180n
M1256 t551 t547 0 0 nch w=1u l=180n
M1257 t549 nd21 vdd vdd pch w=2u l=180n
M1258 t549 t547 vdd vdd pch w=2u l=180n
CT552 t552 0 0.1f
M1259 t549 nd21 t552 0 nch w=1u l=180n
M1260 t552 t547 0 0 nch w=1u l=180n
M1261 nw79 t548 vdd vdd pch w=2u l=180n
M1262 nw79 t549 vdd vdd pch w=2u l=180n
CT553 t553 0 0.1f
M1263 nw79 t548 t553 0 nch w=1u l=180n
M1264 t553 t549 0 0 nch w=1u l=180n
Cnw79 nw79 0 2f
CT554 t554 0 0.1f
CT555 t555 0 0.1f
CT556 t556 0 0.1f
M1265 t554 nw79 vdd vdd pch w=2u l=180n
M1266 t554 nd22 vdd vdd pch w=2u l=180n
CT557 t557 0 0.1f
M1267 t554 nw79 t557 0 nch w=1u l=180n
M1268 t557 nd22 0 0 nch w=1u l=180n
M1269 t555 nw79 vdd vdd pch w=2u l=180n
M1270 t555 t554 vdd vdd pch w=2u l=180n
CT558 t558 0 0.1f
M1271 t555 nw79 t558 0 nch w=1u l=180n
M1272 t558 t554 0 0 nch w=1u l=180n
M1273 t556 nd22 vdd vdd pch w=2u l=180n
M1274 t556 t554 vdd vdd pch w=2u l=180n
CT559 t559 0 0.1f
M1275 t556 nd22 t559 0 nch w=1u l=180n
M1276 t559 t554 0 0 nch w=1u l=180n
M1277 nw80 t555 vdd vdd pch w=2u l=180n
M1278 nw80 t556 vdd vdd pch w=2u l=180n
CT560 t560 0 0.1f
M1279 nw80 t555 t560 0 nch w=1u l=180n
M1280 t560 t556 0 0 nch w=1u l=180n
Cnw80 nw80 0 2f
CT561 t561 0 0.1f
CT562 t562 0 0.1f
CT563 t563 0 0.1f
M1281 t561 nw80 vdd vdd pch w=2u l=180n
M1282 t561 nd23 vdd vdd pch w=2u l=180n
CT564 t564 0 0.1f
M1283 t561 nw80 t564 0 nch w=1u l=180n
M1284 t564 nd23 0 0 nch w=1u l=180n
M1285 t562 nw80 vdd vdd pch w=2u l=180n
M1286 t562 t561 vdd vdd pch w=2u l=180n
CT565 t565 0 0.1f
M1287 t562 nw80 t565 0 nch w=1u l=180n
M1288 t565 t561 0 0 nch w=1u l=180n
M1289 t563 nd23 vdd vdd pch w=2u l=180n
M1290 t563 t561 vdd vdd pch w=2u l=180n
CT566 t566 0 0.1f
M1291 t563 nd23 t566 0 nch w=1u l=180n
M1292 t566 t561 0 0 nch w=1u l=180n
M1293 nw81 t562 vdd vdd pch w=2u l=180n
M1294 nw81 t563 vdd vdd pch w=2u l=180n
CT567 t567 0 0.1f
M1295 nw81 t562 t567 0 nch w=1u l=180n
M1296 t567 t563 0 0 nch w=1u l=180n
Cnw81 nw81 0 2f
CT568 t568 0 0.1f
CT569 t569 0 0.1f
CT570 t570 0 0.1f
M1297 t568 nw81 vdd vdd pch w=2u l=180n
M1298 t568 nd24 vdd vdd pch w=2u l=180n
CT571 t571 0 0.1f
M1299 t568 nw81 t571 0 nch w=1u l=180n
M1300 t571 nd24 0 0 nch w=1u l=180n
M1301 t569 nw81 vdd vdd pch w=2u l=180n
M1302 t569 t568 vdd vdd pch w=2u l=180n
CT572 t572 0 0.1f
M1303 t569 nw81 t572 0 nch w=1u l=180n
M1304 t572 t568 0 0 nch w=1u l=180n
M1305 t570 nd24 vdd vdd pch w=2u l=180n
M1306 t570 t568 vdd vdd pch w=2u l=180n
CT573 t573 0 0.1f
M1307 t570 nd24 t573 0 nch w=1u l=180n
M1308 t573 t568 0 0 nch w=1u l=180n
M1309 nw82 t569 vdd vdd pch w=2u l=180n
M1310 nw82 t570 vdd vdd pch w=2u l=180n
CT574 t574 0 0.1f
M1311 nw82 t569 t574 0 nch w=1u l=180n
M1312 t574 t570 0 0 nch w=1u l=180n
Cnw82 nw82 0 2f
CT575 t575 0 0.1f
CT576 t576 0 0.1f
CT577 t577 0 0.1f
M1313 t575 nw82 vdd vdd pch w=2u l=180n
M1314 t575 nd25 vdd vdd pch w=2u l=180n
CT578 t578 0 0.1f
M1315 t575 nw82 t578 0 nch w=1u l=180n
M1316 t578 nd25 0 0 nch w=1u l=180n
M1317 t576 nw82 vdd vdd pch w=2u l=180n
M1318 t576 t575 vdd vdd pch w=2u l=180n
CT579 t579 0 0.1f
M1319 t576 nw82 t579 0 nch w=1u l=180n
M1320 t579 t575 0 0 nch w=1u l=180n
M1321 t577 nd25 vdd vdd pch w=2u l=180n
M1322 t577 t575 vdd vdd pch w=2u l=180n
CT580 t580 0 0.1f
M1323 t577 nd25 t580 0 nch w=1u l=180n
M1324 t580 t575 0 0 nch w=1u l=180n
M1325 nw83 t576 vdd vdd pch w=2u l=180n
M1326 nw83 t577 vdd vdd pch w=2u l=180n
CT581 t581 0 0.1f
M1327 nw83 t576 t581 0 nch w=1u l=180n
M1328 t581 t577 0 0 nch w=1u l=180n
Cnw83 nw83 0 2f
CT582 t582 0 0.1f
CT583 t583 0 0.1f
CT584 t584 0 0.1f
M1329 t582 nw83 vdd vdd pch w=2u l=180n
M1330 t582 nr4 vdd vdd pch w=2u l=180n
CT585 t585 0 0.1f
M1331 t582 nw83 t585 0 nch w=1u l=180n
M1332 t585 nr4 0 0 nch w=1u l=180n
M1333 t583 nw83 vdd vdd pch w=2u l=180n
M1334 t583 t582 vdd vdd pch w=2u l=180n
CT586 t586 0 0.1f
M1335 t583 nw83 t586 0 nch w=1u l=180n
M1336 t586 t582 0 0 nch w=1u l=180n
M1337 t584 nr4 vdd vdd pch w=2u l=180n
M1338 t584 t582 vdd vdd pch w=2u l=180n
CT587 t587 0 0.1f
M1339 t584 nr4 t587 0 nch w=1u l=180n
M1340 t587 t582 0 0 nch w=1u l=180n
M1341 nw84 t583 vdd vdd pch w=2u l=180n
M1342 nw84 t584 vdd vdd pch w=2u l=180n
CT588 t588 0 0.1f
M1343 nw84 t583 t588 0 nch w=1u l=180n
M1344 t588 t584 0 0 nch w=1u l=180n
Cnw84 nw84 0 2f
CT589 t589 0 0.1f
CT590 t590 0 0.1f
CT591 t591 0 0.1f
M1345 t589 nd26 vdd vdd pch w=2u l=180n
M1346 t589 nd27 vdd vdd pch w=2u l=180n
CT592 t592 0 0.1f
M1347 t589 nd26 t592 0 nch w=1u l=180n
M1348 t592 nd27 0 0 nch w=1u l=180n
M1349 t590 nd26 vdd vdd pch w=2u l=180n
M1350 t590 t589 vdd vdd pch w=2u l=180n
CT593 t593 0 0.1f
M1351 t590 nd26 t593 0 nch w=1u l=180n
M1352 t593 t589 0 0 nch w=1u l=180n
M1353 t591 nd27 vdd vdd pch w=2u l=180n
M1354 t591 t589 vdd vdd pch w=2u l=180n
CT594 t594 0 0.1f
M1355 t591 nd27 t594 0 nch w=1u l=180n
M1356 t594 t589 0 0 nch w=1u l=180n
M1357 nw85 t590 vdd vdd pch w=2u l=180n
M1358 nw85 t591 vdd vdd pch w=2u l=180n
CT595 t595 0 0.1f
M1359 nw85 t590 t595 0 nch w=1u l=180n
M1360 t595 t591 0 0 nch w=1u l=180n
Cnw85 nw85 0 2f
CT596 t596 0 0.1f
CT597 t597 0 0.1f
CT598 t598 0 0.1f
M1361 t596 nw85 vdd vdd pch w=2u l=180n
M1362 t596 nd28 vdd vdd pch w=2u l=180n
CT599 t599 0 0.1f
M1363 t596 nw85 t599 0 nch w=1u l=180n
M1364 t599 nd28 0 0 nch w=1u l=180n
M1365 t597 nw85 vdd vdd pch w=2u l=180n
M1366 t597 t596 vdd vdd pch w=2u l=180n
CT600 t600 0 0.1f
M1367 t597 nw85 t600 0 nch w=1u l=180n
M1368 t600 t596 0 0 nch w=1u l=180n
M1369 t598 nd28 vdd vdd pch w=2u l=180n
M1370 t598 t596 vdd vdd pch w=2u l=180n
CT601 t601 0 0.1f
M1371 t598 nd28 t601 0 nch w=1u l=180n
M1372 t601 t596 0 0 nch w=1u l=180n
M1373 nw86 t597 vdd vdd pch w=2u l=180n
M1374 nw86 t598 vdd vdd pch w=2u l=180n
CT602 t602 0 0.1f
M1375 nw86 t597 t602 0 nch w=1u l=180n
M1376 t602 t598 0 0 nch w=1u l=180n
Cnw86 nw86 0 2f
CT603 t603 0 0.1f
CT604 t604 0 0.1f
CT605 t605 0 0.1f
M1377 t603 nw86 vdd vdd pch w=2u l=180n
M1378 t603 nd29 vdd vdd pch w=2u l=180n
CT606 t606 0 0.1f
M1379 t603 nw86 t606 0 nch w=1u l=180n
M1380 t606 nd29 0 0 nch w=1u l=180n
M1381 t604 nw86 vdd vdd pch w=2u l=180n
M1382 t604 t603 vdd vdd pch w=2u l=180n
CT607 t607 0 0.1f
M1383 t604 nw86 t607 0 nch w=1u l=180n
M1384 t607 t603 0 0 nch w=1u l=180n
M1385 t605 nd29 vdd vdd pch w=2u l=180n
M1386 t605 t603 vdd vdd pch w=2u l=180n
CT608 t608 0 0.1f
M1387 t605 nd29 t608 0 nch w=1u l=180n
M1388 t608 t603 0 0 nch w=1u l=180n
M1389 nw87 t604 vdd vdd pch w=2u l=180n
M1390 nw87 t605 vdd vdd pch w=2u l=180n
CT609 t609 0 0.1f
M1391 nw87 t604 t609 0 nch w=1u l=180n
M1392 t609 t605 0 0 nch w=1u l=180n
Cnw87 nw87 0 2f
CT610 t610 0 0.1f
CT611 t611 0 0.1f
CT612 t612 0 0.1f
M1393 t610 nw87 vdd vdd pch w=2u l=180n
M1394 t610 nd30 vdd vdd pch w=2u l=180n
CT613 t613 0 0.1f
M1395 t610 nw87 t613 0 nch w=1u l=180n
M1396 t613 nd30 0 0 nch w=1u l=180n
M1397 t611 nw87 vdd vdd pch w=2u l=180n
M1398 t611 t610 vdd vdd pch w=2u l=180n
CT614 t614 0 0.1f
M1399 t611 nw87 t614 0 nch w=1u l=180n
M1400 t614 t610 0 0 nch w=1u l=180n
M1401 t612 nd30 vdd vdd pch w=2u l=180n
M1402 t612 t610 vdd vdd pch w=2u l=180n
CT615 t615 0 0.1f
M1403 t612 nd30 t615 0 nch w=1u l=180n
M1404 t615 t610 0 0 nch w=1u l=180n
M1405 nw88 t611 vdd vdd pch w=2u l=180n
M1406 nw88 t612 vdd vdd pch w=2u l=180n
CT616 t616 0 0.1f
M1407 nw88 t611 t616 0 nch w=1u l=180n
M1408 t616 t612 0 0 nch w=1u l=180n
Cnw88 nw88 0 2f
CT617 t617 0 0.1f
CT618 t618 0 0.1f
CT619 t619 0 0.1f
M1409 t617 nw88 vdd vdd pch w=2u l=180n
M1410 t617 nd31 vdd vdd pch w=2u l=180n
CT620 t620 0 0.1f
M1411 t617 nw88 t620 0 nch w=1u l=180n
M1412 t620 nd31 0 0 nch w=1u l=180n
M1413 t618 nw88 vdd vdd pch w=2u l=180n
M1414 t618 t617 vdd vdd pch w=2u l=180n
CT621 t621 0 0.1f
M1415 t618 nw88 t621 0 nch w=1u l=180n
M1416 t621 t617 0 0 nch w=1u l=180n
M1417 t619 nd31 vdd vdd pch w=2u l=180n
M1418 t619 t617 vdd vdd pch w=2u l=180n
CT622 t622 0 0.1f
M1419 t619 nd31 t622 0 nch w=1u l=180n
M1420 t622 t617 0 0 nch w=1u l=180n
M1421 nw89 t618 vdd vdd pch w=2u l=180n
M1422 nw89 t619 vdd vdd pch w=2u l=180n
CT623 t623 0 0.1f
M1423 nw89 t618 t623 0 nch w=1u l=180n
M1424 t623 t619 0 0 nch w=1u l=180n
Cnw89 nw89 0 2f
CT624 t624 0 0.1f
CT625 t625 0 0.1f
CT626 t626 0 0.1f
M1425 t624 nw89 vdd vdd pch w=2u l=180n
M1426 t624 nr5 vdd vdd pch w=2u l=180n
CT627 t627 0 0.1f
M1427 t624 nw89 t627 0 nch w=1u l=180n
M1428 t627 nr5 0 0 nch w=1u l=180n
M1429 t625 nw89 vdd vdd pch w=2u l=180n
M1430 t625 t624 vdd vdd pch w=2u l=180n
CT628 t628 0 0.1f
M1431 t625 nw89 t628 0 nch w=1u l=180n
M1432 t628 t624 0 0 nch w=1u l=180n
M1433 t626 nr5 vdd vdd pch w=2u l=180n
M1434 t626 t624 vdd vdd pch w=2u l=180n
CT629 t629 0 0.1f
M1435 t626 nr5 t629 0 nch w=1u l=180n
M1436 t629 t624 0 0 nch w=1u l=180n
M1437 nw90 t625 vdd vdd pch w=2u l=180n
M1438 nw90 t626 vdd vdd pch w=2u l=180n
CT630 t630 0 0.1f
M1439 nw90 t625 t630 0 nch w=1u l=180n
M1440 t630 t626 0 0 nch w=1u l=180n
Cnw90 nw90 0 2f
M1441 nw91 nw18 vdd vdd pch w=2u l=180n
M1442 nw91 nw18 0 0 nch w=1u l=180n
Cnw91 nw91 0 2f
M1443 nw92 nw36 vdd vdd pch w=2u l=180n
M1444 nw92 nw36 0 0 nch w=1u l=180n
Cnw92 nw92 0 2f
M1445 nw93 nw54 vdd vdd pch w=2u l=180n
M1446 nw93 nw54 0 0 nch w=1u l=180n
Cnw93 nw93 0 2f
M1447 nw94 nw69 vdd vdd pch w=2u l=180n
M1448 nw94 nw69 0 0 nch w=1u l=180n
Cnw94 nw94 0 2f
M1449 nw95 nw84 vdd vdd pch w=2u l=180n
M1450 nw95 nw84 0 0 nch w=1u l=180n
Cnw95 nw95 0 2f
M1451 nw96 nw90 vdd vdd pch w=2u l=180n
M1452 nw96 nw90 0 0 nch w=1u l=180n
Cnw96 nw96 0 2f
CT631 t631 0 0.1f
M1453 t631 nw18 vdd vdd pch w=2u l=180n
M1454 t631 nw36 vdd vdd pch w=2u l=180n
M1455 t631 nw93 vdd vdd pch w=2u l=180n
M1456 t631 nw94 vdd vdd pch w=2u l=180n
M1457 t631 nw95 vdd vdd pch w=2u l=180n
M1458 t631 nw96 vdd vdd pch w=2u l=180n
M1459 t631 nen vdd vdd pch w=2u l=180n
CT632 t632 0 0.1f
M1460 t631 nw18 t632 0 nch w=1u l=180n
CT633 t633 0 0.1f
M1461 t632 nw36 t633 0 nch w=1u l=180n
CT634 t634 0 0.1f
M1462 t633 nw93 t634 0 nch w=1u l=180n
CT635 t635 0 0.1f
M1463 t634 nw94 t635 0 nch w=1u l=180n
CT636 t636 0 0.1f
M1464 t635 nw95 t636 0 nch w=1u l=180n
CT637 t637 0 0.1f
M1465 t636 nw96 t637 0 nch w=1u l=180n
M1466 t637 nen 0 0 nch w=1u l=180n
M1467 nw97 t631 vdd vdd pch w=2u l=180n
M1468 nw97 t631 0 0 nch w=1u l=180n
Cnw97 nw97 0 2f
CT638 t638 0 0.1f
CT639 t639 0 0.1f
CT640 t640 0 0.1f
M1469 t638 nd0 vdd vdd pch w=2u l=180n
M1470 t638 nw97 vdd vdd pch w=2u l=180n
CT641 t641 0 0.1f
M1471 t638 nd0 t641 0 nch w=1u l=180n
M1472 t641 nw97 0 0 nch w=1u l=180n
M1473 t639 nd0 vdd vdd pch w=2u l=180n
M1474 t639 t638 vdd vdd pch w=2u l=180n
CT642 t642 0 0.1f
M1475 t639 nd0 t642 0 nch w=1u l=180n
M1476 t642 t638 0 0 nch w=1u l=180n
M1477 t640 nw97 vdd vdd pch w=2u l=180n
M1478 t640 t638 vdd vdd pch w=2u l=180n
CT643 t643 0 0.1f
M1479 t640 nw97 t643 0 nch w=1u l=180n
M1480 t643 t638 0 0 nch w=1u l=180n
M1481 nw98 t639 vdd vdd pch w=2u l=180n
M1482 nw98 t640 vdd vdd pch w=2u l=180n
CT644 t644 0 0.1f
M1483 nw98 t639 t644 0 nch w=1u l=180n
M1484 t644 t640 0 0 nch w=1u l=180n
Cnw98 nw98 0 2f
CT645 t645 0 0.1f
M1485 t645 nw98 vdd vdd pch w=2u l=180n
M1486 t645 nw98 0 0 nch w=1u l=180n
M1487 nq0 t645 vdd vdd pch w=2u l=180n
M1488 nq0 t645 0 0 nch w=1u l=180n
Cnq0 nq0 0 2f
CT646 t646 0 0.1f
M1489 t646 nw18 vdd vdd pch w=2u l=180n
M1490 t646 nw92 vdd vdd pch w=2u l=180n
M1491 t646 nw54 vdd vdd pch w=2u l=180n
M1492 t646 nw94 vdd vdd pch w=2u l=180n
M1493 t646 nw95 vdd vdd pch w=2u l=180n
M1494 t646 nw96 vdd vdd pch w=2u l=180n
M1495 t646 nen vdd vdd pch w=2u l=180n
CT647 t647 0 0.1f
M1496 t646 nw18 t647 0 nch w=1u l=180n
CT648 t648 0 0.1f
M1497 t647 nw92 t648 0 nch w=1u l=180n
CT649 t649 0 0.1f
M1498 t648 nw54 t649 0 nch w=1u l=180n
CT650 t650 0 0.1f
M1499 t649 nw94 t650 0 nch w=1u l=180n
CT651 t651 0 0.1f
M1500 t650 nw95 t651 0 nch w=1u l=180n
CT652 t652 0 0.1f
M1501 t651 nw96 t652 0 nch w=1u l=180n
M1502 t652 nen 0 0 nch w=1u l=180n
M1503 nw100 t646 vdd vdd pch w=2u l=180n
M1504 nw100 t646 0 0 nch w=1u l=180n
Cnw100 nw100 0 2f
CT653 t653 0 0.1f
CT654 t654 0 0.1f
CT655 t655 0 0.1f
M1505 t653 nd1 vdd vdd pch w=2u l=180n
M1506 t653 nw100 vdd vdd pch w=2u l=180n
CT656 t656 0 0.1f
M1507 t653 nd1 t656 0 nch w=1u l=180n
M1508 t656 nw100 0 0 nch w=1u l=180n
M1509 t654 nd1 vdd vdd pch w=2u l=180n
M1510 t654 t653 vdd vdd pch w=2u l=180n
CT657 t657 0 0.1f
M1511 t654 nd1 t657 0 nch w=1u l=180n
M1512 t657 t653 0 0 nch w=1u l=180n
M1513 t655 nw100 vdd vdd pch w=2u l=180n
M1514 t655 t653 vdd vdd pch w=2u l=180n
CT658 t658 0 0.1f
M1515 t655 nw100 t658 0 nch w=1u l=180n
M1516 t658 t653 0 0 nch w=1u l=180n
M1517 nw101 t654 vdd vdd pch w=2u l=180n
M1518 nw101 t655 vdd vdd pch w=2u l=180n
CT659 t659 0 0.1f
M1519 nw101 t654 t659 0 nch w=1u l=180n
M1520 t659 t655 0 0 nch w=1u l=180n
Cnw101 nw101 0 2f
CT660 t660 0 0.1f
M1521 t660 nw101 vdd vdd pch w=2u l=180n
M1522 t660 nw101 0 0 nch w=1u l=180n
M1523 nq1 t660 vdd vdd pch w=2u l=180n
M1524 nq1 t660 0 0 nch w=1u l=180n
Cnq1 nq1 0 2f
CT661 t661 0 0.1f
M1525 t661 nw91 vdd vdd pch w=2u l=180n
M1526 t661 nw36 vdd vdd pch w=2u l=180n
M1527 t661 nw54 vdd vdd pch w=2u l=180n
M1528 t661 nw94 vdd vdd pch w=2u l=180n
M1529 t661 nw95 vdd vdd pch w=2u l=180n
M1530 t661 nw96 vdd vdd pch w=2u l=180n
M1531 t661 nen vdd vdd pch w=2u l=180n
CT662 t662 0 0.1f
M1532 t661 nw91 t662 0 nch w=1u l=180n
CT663 t663 0 0.1f
M1533 t662 nw36 t663 0 nch w=1u l=180n
CT664 t664 0 0.1f
M1534 t663 nw54 t664 0 nch w=1u l=180n
CT665 t665 0 0.1f
M1535 t664 nw94 t665 0 nch w=1u l=180n
CT666 t666 0 0.1f
M1536 t665 nw95 t666 0 nch w=1u l=180n
CT667 t667 0 0.1f
M1537 t666 nw96 t667 0 nch w=1u l=180n
M1538 t667 nen 0 0 nch w=1u l=180n
M1539 nw103 t661 vdd vdd pch w=2u l=180n
M1540 nw103 t661 0 0 nch w=1u l=180n
Cnw103 nw103 0 2f
CT668 t668 0 0.1f
CT669 t669 0 0.1f
CT670 t670 0 0.1f
M1541 t668 nd2 vdd vdd pch w=2u l=180n
M1542 t668 nw103 vdd vdd pch w=2u l=180n
CT671 t671 0 0.1f
M1543 t668 nd2 t671 0 nch w=1u l=180n
M1544 t671 nw103 0 0 nch w=1u l=180n
M1545 t669 nd2 vdd vdd pch w=2u l=180n
M1546 t669 t668 vdd vdd pch w=2u l=180n
CT672 t672 0 0.1f
M1547 t669 nd2 t672 0 nch w=1u l=180n
M1548 t672 t668 0 0 nch w=1u l=180n
M1549 t670 nw103 vdd vdd pch w=2u l=180n
M1550 t670 t668 vdd vdd pch w=2u l=180n
CT673 t673 0 0.1f
M1551 t670 nw103 t673 0 nch w=1u l=180n
M1552 t673 t668 0 0 nch w=1u l=180n
M1553 nw104 t669 vdd vdd pch w=2u l=180n
M1554 nw104 t670 vdd vdd pch w=2u l=180n
CT674 t674 0 0.1f
M1555 nw104 t669 t674 0 nch w=1u l=180n
M1556 t674 t670 0 0 nch w=1u l=180n
Cnw104 nw104 0 2f
CT675 t675 0 0.1f
M1557 t675 nw104 vdd vdd pch w=2u l=180n
M1558 t675 nw104 0 0 nch w=1u l=180n
M1559 nq2 t675 vdd vdd pch w=2u l=180n
M1560 nq2 t675 0 0 nch w=1u l=180n
Cnq2 nq2 0 2f
CT676 t676 0 0.1f
M1561 t676 nw18 vdd vdd pch w=2u l=180n
M1562 t676 nw36 vdd vdd pch w=2u l=180n
M1563 t676 nw54 vdd vdd pch w=2u l=180n
M1564 t676 nw94 vdd vdd pch w=2u l=180n
M1565 t676 nw95 vdd vdd pch w=2u l=180n
M1566 t676 nw96 vdd vdd pch w=2u l=180n
M1567 t676 nen vdd vdd pch w=2u l=180n
CT677 t677 0 0.1f
M1568 t676 nw18 t677 0 nch w=1u l=180n
CT678 t678 0 0.1f
M1569 t677 nw36 t678 0 nch w=1u l=180n
CT679 t679 0 0.1f
M1570 t678 nw54 t679 0 nch w=1u l=180n
CT680 t680 0 0.1f
M1571 t679 nw94 t680 0 nch w=1u l=180n
CT681 t681 0 0.1f
M1572 t680 nw95 t681 0 nch w=1u l=180n
CT682 t682 0 0.1f
M1573 t681 nw96 t682 0 nch w=1u l=180n
M1574 t682 nen 0 0 nch w=1u l=180n
M1575 nw106 t676 vdd vdd pch w=2u l=180n
M1576 nw106 t676 0 0 nch w=1u l=180n
Cnw106 nw106 0 2f
CT683 t683 0 0.1f
CT684 t684 0 0.1f
CT685 t685 0 0.1f
M1577 t683 nd3 vdd vdd pch w=2u l=180n
M1578 t683 nw106 vdd vdd pch w=2u l=180n
CT686 t686 0 0.1f
M1579 t683 nd3 t686 0 nch w=1u l=180n
M1580 t686 nw106 0 0 nch w=1u l=180n
M1581 t684 nd3 vdd vdd pch w=2u l=180n
M1582 t684 t683 vdd vdd pch w=2u l=180n
CT687 t687 0 0.1f
M1583 t684 nd3 t687 0 nch w=1u l=180n
M1584 t687 t683 0 0 nch w=1u l=180n
M1585 t685 nw106 vdd vdd pch w=2u l=180n
M1586 t685 t683 vdd vdd pch w=2u l=180n
CT688 t688 0 0.1f
M1587 t685 nw106 t688 0 nch w=1u l=180n
M1588 t688 t683 0 0 nch w=1u l=180n
M1589 nw107 t684 vdd vdd pch w=2u l=180n
M1590 nw107 t685 vdd vdd pch w=2u l=180n
CT689 t689 0 0.1f
M1591 nw107 t684 t689 0 nch w=1u l=180n
M1592 t689 t685 0 0 nch w=1u l=180n
Cnw107 nw107 0 2f
CT690 t690 0 0.1f
M1593 t690 nw107 vdd vdd pch w=2u l=180n
M1594 t690 nw107 0 0 nch w=1u l=180n
M1595 nq3 t690 vdd vdd pch w=2u l=180n
M1596 nq3 t690 0 0 nch w=1u l=180n
Cnq3 nq3 0 2f
CT691 t691 0 0.1f
M1597 t691 nw18 vdd vdd pch w=2u l=180n
M1598 t691 nw92 vdd vdd pch w=2u l=180n
M1599 t691 nw93 vdd vdd pch w=2u l=180n
M1600 t691 nw69 vdd vdd pch w=2u l=180n
M1601 t691 nw95 vdd vdd pch w=2u l=180n
M1602 t691 nw96 vdd vdd pch w=2u l=180n
M1603 t691 nen vdd vdd pch w=2u l=180n
CT692 t692 0 0.1f
M1604 t691 nw18 t692 0 nch w=1u l=180n
CT693 t693 0 0.1f
M1605 t692 nw92 t693 0 nch w=1u l=180n
CT694 t694 0 0.1f
M1606 t693 nw93 t694 0 nch w=1u l=180n
CT695 t695 0 0.1f
M1607 t694 nw69 t695 0 nch w=1u l=180n
CT696 t696 0 0.1f
M1608 t695 nw95 t696 0 nch w=1u l=180n
CT697 t697 0 0.1f
M1609 t696 nw96 t697 0 nch w=1u l=180n
M1610 t697 nen 0 0 nch w=1u l=180n
M1611 nw109 t691 vdd vdd pch w=2u l=180n
M1612 nw109 t691 0 0 nch w=1u l=180n
Cnw109 nw109 0 2f
CT698 t698 0 0.1f
CT699 t699 0 0.1f
CT700 t700 0 0.1f
M1613 t698 nd4 vdd vdd pch w=2u l=180n
M1614 t698 nw109 vdd vdd pch w=2u l=180n
CT701 t701 0 0.1f
M1615 t698 nd4 t701 0 nch w=1u l=180n
M1616 t701 nw109 0 0 nch w=1u l=180n
M1617 t699 nd4 vdd vdd pch w=2u l=180n
M1618 t699 t698 vdd vdd pch w=2u l=180n
CT702 t702 0 0.1f
M1619 t699 nd4 t702 0 nch w=1u l=180n
M1620 t702 t698 0 0 nch w=1u l=180n
M1621 t700 nw109 vdd vdd pch w=2u l=180n
M1622 t700 t698 vdd vdd pch w=2u l=180n
CT703 t703 0 0.1f
M1623 t700 nw109 t703 0 nch w=1u l=180n
M1624 t703 t698 0 0 nch w=1u l=180n
M1625 nw110 t699 vdd vdd pch w=2u l=180n
M1626 nw110 t700 vdd vdd pch w=2u l=180n
CT704 t704 0 0.1f
M1627 nw110 t699 t704 0 nch w=1u l=180n
M1628 t704 t700 0 0 nch w=1u l=180n
Cnw110 nw110 0 2f
CT705 t705 0 0.1f
M1629 t705 nw110 vdd vdd pch w=2u l=180n
M1630 t705 nw110 0 0 nch w=1u l=180n
M1631 nq4 t705 vdd vdd pch w=2u l=180n
M1632 nq4 t705 0 0 nch w=1u l=180n
Cnq4 nq4 0 2f
CT706 t706 0 0.1f
M1633 t706 nw91 vdd vdd pch w=2u l=180n
M1634 t706 nw36 vdd vdd pch w=2u l=180n
M1635 t706 nw93 vdd vdd pch w=2u l=180n
M1636 t706 nw69 vdd vdd pch w=2u l=180n
M1637 t706 nw95 vdd vdd pch w=2u l=180n
M1638 t706 nw96 vdd vdd pch w=2u l=180n
M1639 t706 nen vdd vdd pch w=2u l=180n
CT707 t707 0 0.1f
M1640 t706 nw91 t707 0 nch w=1u l=180n
CT708 t708 0 0.1f
M1641 t707 nw36 t708 0 nch w=1u l=180n
CT709 t709 0 0.1f
M1642 t708 nw93 t709 0 nch w=1u l=180n
CT710 t710 0 0.1f
M1643 t709 nw69 t710 0 nch w=1u l=180n
CT711 t711 0 0.1f
M1644 t710 nw95 t711 0 nch w=1u l=180n
CT712 t712 0 0.1f
M1645 t711 nw96 t712 0 nch w=1u l=180n
M1646 t712 nen 0 0 nch w=1u l=180n
M1647 nw112 t706 vdd vdd pch w=2u l=180n
M1648 nw112 t706 0 0 nch w=1u l=180n
Cnw112 nw112 0 2f
CT713 t713 0 0.1f
CT714 t714 0 0.1f
CT715 t715 0 0.1f
M1649 t713 nd5 vdd vdd pch w=2u l=180n
M1650 t713 nw112 vdd vdd pch w=2u l=180n
CT716 t716 0 0.1f
M1651 t713 nd5 t716 0 nch w=1u l=180n
M1652 t716 nw112 0 0 nch w=1u l=180n
M1653 t714 nd5 vdd vdd pch w=2u l=180n
M1654 t714 t713 vdd vdd pch w=2u l=180n
CT717 t717 0 0.1f
M1655 t714 nd5 t717 0 nch w=1u l=180n
M1656 t717 t713 0 0 nch w=1u l=180n
M1657 t715 nw112 vdd vdd pch w=2u l=180n
M1658 t715 t713 vdd vdd pch w=2u l=180n
CT718 t718 0 0.1f
M1659 t715 nw112 t718 0 nch w=1u l=180n
M1660 t718 t713 0 0 nch w=1u l=180n
M1661 nw113 t714 vdd vdd pch w=2u l=180n
M1662 nw113 t715 vdd vdd pch w=2u l=180n
CT719 t719 0 0.1f
M1663 nw113 t714 t719 0 nch w=1u l=180n
M1664 t719 t715 0 0 nch w=1u l=180n
Cnw113 nw113 0 2f
CT720 t720 0 0.1f
M1665 t720 nw113 vdd vdd pch w=2u l=180n
M1666 t720 nw113 0 0 nch w=1u l=180n
M1667 nq5 t720 vdd vdd pch w=2u l=180n
M1668 nq5 t720 0 0 nch w=1u l=180n
Cnq5 nq5 0 2f
CT721 t721 0 0.1f
M1669 t721 nw18 vdd vdd pch w=2u l=180n
M1670 t721 nw36 vdd vdd pch w=2u l=180n
M1671 t721 nw93 vdd vdd pch w=2u l=180n
M1672 t721 nw69 vdd vdd pch w=2u l=180n
M1673 t721 nw95 vdd vdd pch w=2u l=180n
M1674 t721 nw96 vdd vdd pch w=2u l=180n
M1675 t721 nen vdd vdd pch w=2u l=180n
CT722 t722 0 0.1f
M1676 t721 nw18 t722 0 nch w=1u l=180n
CT723 t723 0 0.1f
M1677 t722 nw36 t723 0 nch w=1u l=180n
CT724 t724 0 0.1f
M1678 t723 nw93 t724 0 nch w=1u l=180n
CT725 t725 0 0.1f
M1679 t724 nw69 t725 0 nch w=1u l=180n
CT726 t726 0 0.1f
M1680 t725 nw95 t726 0 nch w=1u l=180n
CT727 t727 0 0.1f
M1681 t726 nw96 t727 0 nch w=1u l=180n
M1682 t727 nen 0 0 nch w=1u l=180n
M1683 nw115 t721 vdd vdd pch w=2u l=180n
M1684 nw115 t721 0 0 nch w=1u l=180n
Cnw115 nw115 0 2f
CT728 t728 0 0.1f
CT729 t729 0 0.1f
CT730 t730 0 0.1f
M1685 t728 nd6 vdd vdd pch w=2u l=180n
M1686 t728 nw115 vdd vdd pch w=2u l=180n
CT731 t731 0 0.1f
M1687 t728 nd6 t731 0 nch w=1u l=180n
M1688 t731 nw115 0 0 nch w=1u l=180n
M1689 t729 nd6 vdd vdd pch w=2u l=180n
M1690 t729 t728 vdd vdd pch w=2u l=180n
CT732 t732 0 0.1f
M1691 t729 nd6 t732 0 nch w=1u l=180n
M1692 t732 t728 0 0 nch w=1u l=180n
M1693 t730 nw115 vdd vdd pch w=2u l=180n
M1694 t730 t728 vdd vdd pch w=2u l=180n
CT733 t733 0 0.1f
M1695 t730 nw115 t733 0 nch w=1u l=180n
M1696 t733 t728 0 0 nch w=1u l=180n
M1697 nw116 t729 vdd vdd pch w=2u l=180n
M1698 nw116 t730 vdd vdd pch w=2u l=180n
CT734 t734 0 0.1f
M1699 nw116 t729 t734 0 nch w=1u l=180n
M1700 t734 t730 0 0 nch w=1u l=180n
Cnw116 nw116 0 2f
CT735 t735 0 0.1f
M1701 t735 nw116 vdd vdd pch w=2u l=180n
M1702 t735 nw116 0 0 nch w=1u l=180n
M1703 nq6 t735 vdd vdd pch w=2u l=180n
M1704 nq6 t735 0 0 nch w=1u l=180n
Cnq6 nq6 0 2f
CT736 t736 0 0.1f
M1705 t736 nw91 vdd vdd pch w=2u l=180n
M1706 t736 nw92 vdd vdd pch w=2u l=180n
M1707 t736 nw54 vdd vdd pch w=2u l=180n
M1708 t736 nw69 vdd vdd pch w=2u l=180n
M1709 t736 nw95 vdd vdd pch w=2u l=180n
M1710 t736 nw96 vdd vdd pch w=2u l=180n
M1711 t736 nen vdd vdd pch w=2u l=180n
CT737 t737 0 0.1f
M1712 t736 nw91 t737 0 nch w=1u l=180n
CT738 t738 0 0.1f
M1713 t737 nw92 t738 0 nch w=1u l=180n
CT739 t739 0 0.1f
M1714 t738 nw54 t739 0 nch w=1u l=180n
CT740 t740 0 0.1f
M1715 t739 nw69 t740 0 nch w=1u l=180n
CT741 t741 0 0.1f
M1716 t740 nw95 t741 0 nch w=1u l=180n
CT742 t742 0 0.1f
M1717 t741 nw96 t742 0 nch w=1u l=180n
M1718 t742 nen 0 0 nch w=1u l=180n
M1719 nw118 t736 vdd vdd pch w=2u l=180n
M1720 nw118 t736 0 0 nch w=1u l=180n
Cnw118 nw118 0 2f
CT743 t743 0 0.1f
CT744 t744 0 0.1f
CT745 t745 0 0.1f
M1721 t743 nd7 vdd vdd pch w=2u l=180n
M1722 t743 nw118 vdd vdd pch w=2u l=180n
CT746 t746 0 0.1f
M1723 t743 nd7 t746 0 nch w=1u l=180n
M1724 t746 nw118 0 0 nch w=1u l=180n
M1725 t744 nd7 vdd vdd pch w=2u l=180n
M1726 t744 t743 vdd vdd pch w=2u l=180n
CT747 t747 0 0.1f
M1727 t744 nd7 t747 0 nch w=1u l=180n
M1728 t747 t743 0 0 nch w=1u l=180n
M1729 t745 nw118 vdd vdd pch w=2u l=180n
M1730 t745 t743 vdd vdd pch w=2u l=180n
CT748 t748 0 0.1f
M1731 t745 nw118 t748 0 nch w=1u l=180n
M1732 t748 t743 0 0 nch w=1u l=180n
M1733 nw119 t744 vdd vdd pch w=2u l=180n
M1734 nw119 t745 vdd vdd pch w=2u l=180n
CT749 t749 0 0.1f
M1735 nw119 t744 t749 0 nch w=1u l=180n
M1736 t749 t745 0 0 nch w=1u l=180n
Cnw119 nw119 0 2f
CT750 t750 0 0.1f
M1737 t750 nw119 vdd vdd pch w=2u l=180n
M1738 t750 nw119 0 0 nch w=1u l=180n
M1739 nq7 t750 vdd vdd pch w=2u l=180n
M1740 nq7 t750 0 0 nch w=1u l=180n
Cnq7 nq7 0 2f
CT751 t751 0 0.1f
M1741 t751 nw18 vdd vdd pch w=2u l=180n
M1742 t751 nw92 vdd vdd pch w=2u l=180n
M1743 t751 nw54 vdd vdd pch w=2u l=180n
M1744 t751 nw69 vdd vdd pch w=2u l=180n
M1745 t751 nw95 vdd vdd pch w=2u l=180n
M1746 t751 nw96 vdd vdd pch w=2u l=180n
M1747 t751 nen vdd vdd pch w=2u l=180n
CT752 t752 0 0.1f
M1748 t751 nw18 t752 0 nch w=1u l=180n
CT753 t753 0 0.1f
M1749 t752 nw92 t753 0 nch w=1u l=180n
CT754 t754 0 0.1f
M1750 t753 nw54 t754 0 nch w=1u l=180n
CT755 t755 0 0.1f
M1751 t754 nw69 t755 0 nch w=1u l=180n
CT756 t756 0 0.1f
M1752 t755 nw95 t756 0 nch w=1u l=180n
CT757 t757 0 0.1f
M1753 t756 nw96 t757 0 nch w=1u l=180n
M1754 t757 nen 0 0 nch w=1u l=180n
M1755 nw121 t751 vdd vdd pch w=2u l=180n
M1756 nw121 t751 0 0 nch w=1u l=180n
Cnw121 nw121 0 2f
CT758 t758 0 0.1f
CT759 t759 0 0.1f
CT760 t760 0 0.1f
M1757 t758 nd8 vdd vdd pch w=2u l=180n
M1758 t758 nw121 vdd vdd pch w=2u l=180n
CT761 t761 0 0.1f
M1759 t758 nd8 t761 0 nch w=1u l=180n
M1760 t761 nw121 0 0 nch w=1u l=180n
M1761 t759 nd8 vdd vdd pch w=2u l=180n
M1762 t759 t758 vdd vdd pch w=2u l=180n
CT762 t762 0 0.1f
M1763 t759 nd8 t762 0 nch w=1u l=180n
M1764 t762 t758 0 0 nch w=1u l=180n
M1765 t760 nw121 vdd vdd pch w=2u l=180n
M1766 t760 t758 vdd vdd pch w=2u l=180n
CT763 t763 0 0.1f
M1767 t760 nw121 t763 0 nch w=1u l=180n
M1768 t763 t758 0 0 nch w=1u l=180n
M1769 nw122 t759 vdd vdd pch w=2u l=180n
M1770 nw122 t760 vdd vdd pch w=2u l=180n
CT764 t764 0 0.1f
M1771 nw122 t759 t764 0 nch w=1u l=180n
M1772 t764 t760 0 0 nch w=1u l=180n
Cnw122 nw122 0 2f
CT765 t765 0 0.1f
M1773 t765 nw122 vdd vdd pch w=2u l=180n
M1774 t765 nw122 0 0 nch w=1u l=180n
M1775 nq8 t765 vdd vdd pch w=2u l=180n
M1776 nq8 t765 0 0 nch w=1u l=180n
Cnq8 nq8 0 2f
CT766 t766 0 0.1f
M1777 t766 nw91 vdd vdd pch w=2u l=180n
M1778 t766 nw36 vdd vdd pch w=2u l=180n
M1779 t766 nw54 vdd vdd pch w=2u l=180n
M1780 t766 nw69 vdd vdd pch w=2u l=180n
M1781 t766 nw95 vdd vdd pch w=2u l=180n
M1782 t766 nw96 vdd vdd pch w=2u l=180n
M1783 t766 nen vdd vdd pch w=2u l=180n
CT767 t767 0 0.1f
M1784 t766 nw91 t767 0 nch w=1u l=180n
CT768 t768 0 0.1f
M1785 t767 nw36 t768 0 nch w=1u l=180n
CT769 t769 0 0.1f
M1786 t768 nw54 t769 0 nch w=1u l=180n
CT770 t770 0 0.1f
M1787 t769 nw69 t770 0 nch w=1u l=180n
CT771 t771 0 0.1f
M1788 t770 nw95 t771 0 nch w=1u l=180n
CT772 t772 0 0.1f
M1789 t771 nw96 t772 0 nch w=1u l=180n
M1790 t772 nen 0 0 nch w=1u l=180n
M1791 nw124 t766 vdd vdd pch w=2u l=180n
M1792 nw124 t766 0 0 nch w=1u l=180n
Cnw124 nw124 0 2f
CT773 t773 0 0.1f
CT774 t774 0 0.1f
CT775 t775 0 0.1f
M1793 t773 nd9 vdd vdd pch w=2u l=180n
M1794 t773 nw124 vdd vdd pch w=2u l=180n
CT776 t776 0 0.1f
M1795 t773 nd9 t776 0 nch w=1u l=180n
M1796 t776 nw124 0 0 nch w=1u l=180n
M1797 t774 nd9 vdd vdd pch w=2u l=180n
M1798 t774 t773 vdd vdd pch w=2u l=180n
CT777 t777 0 0.1f
M1799 t774 nd9 t777 0 nch w=1u l=180n
M1800 t777 t773 0 0 nch w=1u l=180n
M1801 t775 nw124 vdd vdd pch w=2u l=180n
M1802 t775 t773 vdd vdd pch w=2u l=180n
CT778 t778 0 0.1f
M1803 t775 nw124 t778 0 nch w=1u l=180n
M1804 t778 t773 0 0 nch w=1u l=180n
M1805 nw125 t774 vdd vdd pch w=2u l=180n
M1806 nw125 t775 vdd vdd pch w=2u l=180n
CT779 t779 0 0.1f
M1807 nw125 t774 t779 0 nch w=1u l=180n
M1808 t779 t775 0 0 nch w=1u l=180n
Cnw125 nw125 0 2f
CT780 t780 0 0.1f
M1809 t780 nw125 vdd vdd pch w=2u l=180n
M1810 t780 nw125 0 0 nch w=1u l=180n
M1811 nq9 t780 vdd vdd pch w=2u l=180n
M1812 nq9 t780 0 0 nch w=1u l=180n
Cnq9 nq9 0 2f
CT781 t781 0 0.1f
M1813 t781 nw18 vdd vdd pch w=2u l=180n
M1814 t781 nw36 vdd vdd pch w=2u l=180n
M1815 t781 nw54 vdd vdd pch w=2u l=180n
M1816 t781 nw69 vdd vdd pch w=2u l=180n
M1817 t781 nw95 vdd vdd pch w=2u l=180n
M1818 t781 nw96 vdd vdd pch w=2u l=180n
M1819 t781 nen vdd vdd pch w=2u l=180n
CT782 t782 0 0.1f
M1820 t781 nw18 t782 0 nch w=1u l=180n
CT783 t783 0 0.1f
M1821 t782 nw36 t783 0 nch w=1u l=180n
CT784 t784 0 0.1f
M1822 t783 nw54 t784 0 nch w=1u l=180n
CT785 t785 0 0.1f
M1823 t784 nw69 t785 0 nch w=1u l=180n
CT786 t786 0 0.1f
M1824 t785 nw95 t786 0 nch w=1u l=180n
CT787 t787 0 0.1f
M1825 t786 nw96 t787 0 nch w=1u l=180n
M1826 t787 nen 0 0 nch w=1u l=180n
M1827 nw127 t781 vdd vdd pch w=2u l=180n
M1828 nw127 t781 0 0 nch w=1u l=180n
Cnw127 nw127 0 2f
CT788 t788 0 0.1f
CT789 t789 0 0.1f
CT790 t790 0 0.1f
M1829 t788 nd10 vdd vdd pch w=2u l=180n
M1830 t788 nw127 vdd vdd pch w=2u l=180n
CT791 t791 0 0.1f
M1831 t788 nd10 t791 0 nch w=1u l=180n
M1832 t791 nw127 0 0 nch w=1u l=180n
M1833 t789 nd10 vdd vdd pch w=2u l=180n
M1834 t789 t788 vdd vdd pch w=2u l=180n
CT792 t792 0 0.1f
M1835 t789 nd10 t792 0 nch w=1u l=180n
M1836 t792 t788 0 0 nch w=1u l=180n
M1837 t790 nw127 vdd vdd pch w=2u l=180n
M1838 t790 t788 vdd vdd pch w=2u l=180n
CT793 t793 0 0.1f
M1839 t790 nw127 t793 0 nch w=1u l=180n
M1840 t793 t788 0 0 nch w=1u l=180n
M1841 nw128 t789 vdd vdd pch w=2u l=180n
M1842 nw128 t790 vdd vdd pch w=2u l=180n
CT794 t794 0 0.1f
M1843 nw128 t789 t794 0 nch w=1u l=180n
M1844 t794 t790 0 0 nch w=1u l=180n
Cnw128 nw128 0 2f
CT795 t795 0 0.1f
M1845 t795 nw128 vdd vdd pch w=2u l=180n
M1846 t795 nw128 0 0 nch w=1u l=180n
M1847 nq10 t795 vdd vdd pch w=2u l=180n
M1848 nq10 t795 0 0 nch w=1u l=180n
Cnq10 nq10 0 2f
CT796 t796 0 0.1f
M1849 t796 nw18 vdd vdd pch w=2u l=180n
M1850 t796 nw92 vdd vdd pch w=2u l=180n
M1851 t796 nw93 vdd vdd pch w=2u l=180n
M1852 t796 nw94 vdd vdd pch w=2u l=180n
M1853 t796 nw84 vdd vdd pch w=2u l=180n
M1854 t796 nw96 vdd vdd pch w=2u l=180n
M1855 t796 nen vdd vdd pch w=2u l=180n
CT797 t797 0 0.1f
M1856 t796 nw18 t797 0 nch w=1u l=180n
CT798 t798 0 0.1f
M1857 t797 nw92 t798 0 nch w=1u l=180n
CT799 t799 0 0.1f
M1858 t798 nw93 t799 0 nch w=1u l=180n
CT800 t800 0 0.1f
M1859 t799 nw94 t800 0 nch w=1u l=180n
CT801 t801 0 0.1f
M1860 t800 nw84 t801 0 nch w=1u l=180n
CT802 t802 0 0.1f
M1861 t801 nw96 t802 0 nch w=1u l=180n
M1862 t802 nen 0 0 nch w=1u l=180n
M1863 nw130 t796 vdd vdd pch w=2u l=180n
M1864 nw130 t796 0 0 nch w=1u l=180n
Cnw130 nw130 0 2f
CT803 t803 0 0.1f
CT804 t804 0 0.1f
CT805 t805 0 0.1f
M1865 t803 nd11 vdd vdd pch w=2u l=180n
M1866 t803 nw130 vdd vdd pch w=2u l=180n
CT806 t806 0 0.1f
M1867 t803 nd11 t806 0 nch w=1u l=180n
M1868 t806 nw130 0 0 nch w=1u l=180n
M1869 t804 nd11 vdd vdd pch w=2u l=180n
M1870 t804 t803 vdd vdd pch w=2u l=180n
CT807 t807 0 0.1f
M1871 t804 nd11 t807 0 nch w=1u l=180n
M1872 t807 t803 0 0 nch w=1u l=180n
M1873 t805 nw130 vdd vdd pch w=2u l=180n
M1874 t805 t803 vdd vdd pch w=2u l=180n
CT808 t808 0 0.1f
M1875 t805 nw130 t808 0 nch w=1u l=180n
M1876 t808 t803 0 0 nch w=1u l=180n
M1877 nw131 t804 vdd vdd pch w=2u l=180n
M1878 nw131 t805 vdd vdd pch w=2u l=180n
CT809 t809 0 0.1f
M1879 nw131 t804 t809 0 nch w=1u l=180n
M1880 t809 t805 0 0 nch w=1u l=180n
Cnw131 nw131 0 2f
CT810 t810 0 0.1f
M1881 t810 nw131 vdd vdd pch w=2u l=180n
M1882 t810 nw131 0 0 nch w=1u l=180n
M1883 nq11 t810 vdd vdd pch w=2u l=180n
M1884 nq11 t810 0 0 nch w=1u l=180n
Cnq11 nq11 0 2f
CT811 t811 0 0.1f
M1885 t811 nw91 vdd vdd pch w=2u l=180n
M1886 t811 nw36 vdd vdd pch w=2u l=180n
M1887 t811 nw93 vdd vdd pch w=2u l=180n
M1888 t811 nw94 vdd vdd pch w=2u l=180n
M1889 t811 nw84 vdd vdd pch w=2u l=180n
M1890 t811 nw96 vdd vdd pch w=2u l=180n
M1891 t811 nen vdd vdd pch w=2u l=180n
CT812 t812 0 0.1f
M1892 t811 nw91 t812 0 nch w=1u l=180n
CT813 t813 0 0.1f
M1893 t812 nw36 t813 0 nch w=1u l=180n
CT814 t814 0 0.1f
M1894 t813 nw93 t814 0 nch w=1u l=180n
CT815 t815 0 0.1f
M1895 t814 nw94 t815 0 nch w=1u l=180n
CT816 t816 0 0.1f
M1896 t815 nw84 t816 0 nch w=1u l=180n
CT817 t817 0 0.1f
M1897 t816 nw96 t817 0 nch w=1u l=180n
M1898 t817 nen 0 0 nch w=1u l=180n
M1899 nw133 t811 vdd vdd pch w=2u l=180n
M1900 nw133 t811 0 0 nch w=1u l=180n
Cnw133 nw133 0 2f
CT818 t818 0 0.1f
CT819 t819 0 0.1f
CT820 t820 0 0.1f
M1901 t818 nd12 vdd vdd pch w=2u l=180n
M1902 t818 nw133 vdd vdd pch w=2u l=180n
CT821 t821 0 0.1f
M1903 t818 nd12 t821 0 nch w=1u l=180n
M1904 t821 nw133 0 0 nch w=1u l=180n
M1905 t819 nd12 vdd vdd pch w=2u l=180n
M1906 t819 t818 vdd vdd pch w=2u l=180n
CT822 t822 0 0.1f
M1907 t819 nd12 t822 0 nch w=1u l=180n
M1908 t822 t818 0 0 nch w=1u l=180n
M1909 t820 nw133 vdd vdd pch w=2u l=180n
M1910 t820 t818 vdd vdd pch w=2u l=180n
CT823 t823 0 0.1f
M1911 t820 nw133 t823 0 nch w=1u l=180n
M1912 t823 t818 0 0 nch w=1u l=180n
M1913 nw134 t819 vdd vdd pch w=2u l=180n
M1914 nw134 t820 vdd vdd pch w=2u l=180n
CT824 t824 0 0.1f
M1915 nw134 t819 t824 0 nch w=1u l=180n
M1916 t824 t820 0 0 nch w=1u l=180n
Cnw134 nw134 0 2f
CT825 t825 0 0.1f
M1917 t825 nw134 vdd vdd pch w=2u l=180n
M1918 t825 nw134 0 0 nch w=1u l=180n
M1919 nq12 t825 vdd vdd pch w=2u l=180n
M1920 nq12 t825 0 0 nch w=1u l=180n
Cnq12 nq12 0 2f
CT826 t826 0 0.1f
M1921 t826 nw18 vdd vdd pch w=2u l=180n
M1922 t826 nw36 vdd vdd pch w=2u l=180n
M1923 t826 nw93 vdd vdd pch w=2u l=180n
M1924 t826 nw94 vdd vdd pch w=2u l=180n
M1925 t826 nw84 vdd vdd pch w=2u l=180n
M1926 t826 nw96 vdd vdd pch w=2u l=180n
M1927 t826 nen vdd vdd pch w=2u l=180n
CT827 t827 0 0.1f
M1928 t826 nw18 t827 0 nch w=1u l=180n
CT828 t828 0 0.1f
M1929 t827 nw36 t828 0 nch w=1u l=180n
CT829 t829 0 0.1f
M1930 t828 nw93 t829 0 nch w=1u l=180n
CT830 t830 0 0.1f
M1931 t829 nw94 t830 0 nch w=1u l=180n
CT831 t831 0 0.1f
M1932 t830 nw84 t831 0 nch w=1u l=180n
CT832 t832 0 0.1f
M1933 t831 nw96 t832 0 nch w=1u l=180n
M1934 t832 nen 0 0 nch w=1u l=180n
M1935 nw136 t826 vdd vdd pch w=2u l=180n
M1936 nw136 t826 0 0 nch w=1u l=180n
Cnw136 nw136 0 2f
CT833 t833 0 0.1f
CT834 t834 0 0.1f
CT835 t835 0 0.1f
M1937 t833 nd13 vdd vdd pch w=2u l=180n
M1938 t833 nw136 vdd vdd pch w=2u l=180n
CT836 t836 0 0.1f
M1939 t833 nd13 t836 0 nch w=1u l=180n
M1940 t836 nw136 0 0 nch w=1u l=180n
M1941 t834 nd13 vdd vdd pch w=2u l=180n
M1942 t834 t833 vdd vdd pch w=2u l=180n
CT837 t837 0 0.1f
M1943 t834 nd13 t837 0 nch w=1u l=180n
M1944 t837 t833 0 0 nch w=1u l=180n
M1945 t835 nw136 vdd vdd pch w=2u l=180n
M1946 t835 t833 vdd vdd pch w=2u l=180n
CT838 t838 0 0.1f
M1947 t835 nw136 t838 0 nch w=1u l=180n
M1948 t838 t833 0 0 nch w=1u l=180n
M1949 nw137 t834 vdd vdd pch w=2u l=180n
M1950 nw137 t835 vdd vdd pch w=2u l=180n
CT839 t839 0 0.1f
M1951 nw137 t834 t839 0 nch w=1u l=180n
M1952 t839 t835 0 0 nch w=1u l=180n
Cnw137 nw137 0 2f
CT840 t840 0 0.1f
M1953 t840 nw137 vdd vdd pch w=2u l=180n
M1954 t840 nw137 0 0 nch w=1u l=180n
M1955 nq13 t840 vdd vdd pch w=2u l=180n
M1956 nq13 t840 0 0 nch w=1u l=180n
Cnq13 nq13 0 2f
CT841 t841 0 0.1f
M1957 t841 nw91 vdd vdd pch w=2u l=180n
M1958 t841 nw92 vdd vdd pch w=2u l=180n
M1959 t841 nw54 vdd vdd pch w=2u l=180n
M1960 t841 nw94 vdd vdd pch w=2u l=180n
M1961 t841 nw84 vdd vdd pch w=2u l=180n
M1962 t841 nw96 vdd vdd pch w=2u l=180n
M1963 t841 nen vdd vdd pch w=2u l=180n
CT842 t842 0 0.1f
M1964 t841 nw91 t842 0 nch w=1u l=180n
CT843 t843 0 0.1f
M1965 t842 nw92 t843 0 nch w=1u l=180n
CT844 t844 0 0.1f
M1966 t843 nw54 t844 0 nch w=1u l=180n
CT845 t845 0 0.1f
M1967 t844 nw94 t845 0 nch w=1u l=180n
CT846 t846 0 0.1f
M1968 t845 nw84 t846 0 nch w=1u l=180n
CT847 t847 0 0.1f
M1969 t846 nw96 t847 0 nch w=1u l=180n
M1970 t847 nen 0 0 nch w=1u l=180n
M1971 nw139 t841 vdd vdd pch w=2u l=180n
M1972 nw139 t841 0 0 nch w=1u l=180n
Cnw139 nw139 0 2f
CT848 t848 0 0.1f
CT849 t849 0 0.1f
CT850 t850 0 0.1f
M1973 t848 nd14 vdd vdd pch w=2u l=180n
M1974 t848 nw139 vdd vdd pch w=2u l=180n
CT851 t851 0 0.1f
M1975 t848 nd14 t851 0 nch w=1u l=180n
M1976 t851 nw139 0 0 nch w=1u l=180n
M1977 t849 nd14 vdd vdd pch w=2u l=180n
M1978 t849 t848 vdd vdd pch w=2u l=180n
CT852 t852 0 0.1f
M1979 t849 nd14 t852 0 nch w=1u l=180n
M1980 t852 t848 0 0 nch w=1u l=180n
M1981 t850 nw139 vdd vdd pch w=2u l=180n
M1982 t850 t848 vdd vdd pch w=2u l=180n
CT853 t853 0 0.1f
M1983 t850 nw139 t853 0 nch w=1u l=180n
M1984 t853 t848 0 0 nch w=1u l=180n
M1985 nw140 t849 vdd vdd pch w=2u l=180n
M1986 nw140 t850 vdd vdd pch w=2u l=180n
CT854 t854 0 0.1f
M1987 nw140 t849 t854 0 nch w=1u l=180n
M1988 t854 t850 0 0 nch w=1u l=180n
Cnw140 nw140 0 2f
CT855 t855 0 0.1f
M1989 t855 nw140 vdd vdd pch w=2u l=180n
M1990 t855 nw140 0 0 nch w=1u l=180n
M1991 nq14 t855 vdd vdd pch w=2u l=180n
M1992 nq14 t855 0 0 nch w=1u l=180n
Cnq14 nq14 0 2f
CT856 t856 0 0.1f
M1993 t856 nw18 vdd vdd pch w=2u l=180n
M1994 t856 nw92 vdd vdd pch w=2u l=180n
M1995 t856 nw54 vdd vdd pch w=2u l=180n
M1996 t856 nw94 vdd vdd pch w=2u l=180n
M1997 t856 nw84 vdd vdd pch w=2u l=180n
M1998 t856 nw96 vdd vdd pch w=2u l=180n
M1999 t856 nen vdd vdd pch w=2u l=180n
CT857 t857 0 0.1f
M2000 t856 nw18 t857 0 nch w=1u l=180n
CT858 t858 0 0.1f
M2001 t857 nw92 t858 0 nch w=1u l=180n
CT859 t859 0 0.1f
M2002 t858 nw54 t859 0 nch w=1u l=180n
CT860 t860 0 0.1f
M2003 t859 nw94 t860 0 nch w=1u l=180n
CT861 t861 0 0.1f
M2004 t860 nw84 t861 0 nch w=1u l=180n
CT862 t862 0 0.1f
M2005 t861 nw96 t862 0 nch w=1u l=180n
M2006 t862 nen 0 0 nch w=1u l=180n
M2007 nw142 t856 vdd vdd pch w=2u l=180n
M2008 nw142 t856 0 0 nch w=1u l=180n
Cnw142 nw142 0 2f
CT863 t863 0 0.1f
CT864 t864 0 0.1f
CT865 t865 0 0.1f
M2009 t863 nd15 vdd vdd pch w=2u l=180n
M2010 t863 nw142 vdd vdd pch w=2u l=180n
CT866 t866 0 0.1f
M2011 t863 nd15 t866 0 nch w=1u l=180n
M2012 t866 nw142 0 0 nch w=1u l=180n
M2013 t864 nd15 vdd vdd pch w=2u l=180n
M2014 t864 t863 vdd vdd pch w=2u l=180n
CT867 t867 0 0.1f
M2015 t864 nd15 t867 0 nch w=1u l=180n
M2016 t867 t863 0 0 nch w=1u l=180n
M2017 t865 nw142 vdd vdd pch w=2u l=180n
M2018 t865 t863 vdd vdd pch w=2u l=180n
CT868 t868 0 0.1f
M2019 t865 nw142 t868 0 nch w=1u l=180n
M2020 t868 t863 0 0 nch w=1u l=180n
M2021 nw143 t864 vdd vdd pch w=2u l=180n
M2022 nw143 t865 vdd vdd pch w=2u l=180n
CT869 t869 0 0.1f
M2023 nw143 t864 t869 0 nch w=1u l=180n
M2024 t869 t865 0 0 nch w=1u l=180n
Cnw143 nw143 0 2f
CT870 t870 0 0.1f
M2025 t870 nw143 vdd vdd pch w=2u l=180n
M2026 t870 nw143 0 0 nch w=1u l=180n
M2027 nq15 t870 vdd vdd pch w=2u l=180n
M2028 nq15 t870 0 0 nch w=1u l=180n
Cnq15 nq15 0 2f
CT871 t871 0 0.1f
M2029 t871 nw91 vdd vdd pch w=2u l=180n
M2030 t871 nw36 vdd vdd pch w=2u l=180n
M2031 t871 nw54 vdd vdd pch w=2u l=180n
M2032 t871 nw94 vdd vdd pch w=2u l=180n
M2033 t871 nw84 vdd vdd pch w=2u l=180n
M2034 t871 nw96 vdd vdd pch w=2u l=180n
M2035 t871 nen vdd vdd pch w=2u l=180n
CT872 t872 0 0.1f
M2036 t871 nw91 t872 0 nch w=1u l=180n
CT873 t873 0 0.1f
M2037 t872 nw36 t873 0 nch w=1u l=180n
CT874 t874 0 0.1f
M2038 t873 nw54 t874 0 nch w=1u l=180n
CT875 t875 0 0.1f
M2039 t874 nw94 t875 0 nch w=1u l=180n
CT876 t876 0 0.1f
M2040 t875 nw84 t876 0 nch w=1u l=180n
CT877 t877 0 0.1f
M2041 t876 nw96 t877 0 nch w=1u l=180n
M2042 t877 nen 0 0 nch w=1u l=180n
M2043 nw145 t871 vdd vdd pch w=2u l=180n
M2044 nw145 t871 0 0 nch w=1u l=180n
Cnw145 nw145 0 2f
CT878 t878 0 0.1f
CT879 t879 0 0.1f
CT880 t880 0 0.1f
M2045 t878 nd16 vdd vdd pch w=2u l=180n
M2046 t878 nw145 vdd vdd pch w=2u l=180n
CT881 t881 0 0.1f
M2047 t878 nd16 t881 0 nch w=1u l=180n
M2048 t881 nw145 0 0 nch w=1u l=180n
M2049 t879 nd16 vdd vdd pch w=2u l=180n
M2050 t879 t878 vdd vdd pch w=2u l=180n
CT882 t882 0 0.1f
M2051 t879 nd16 t882 0 nch w=1u l=180n
M2052 t882 t878 0 0 nch w=1u l=180n
M2053 t880 nw145 vdd vdd pch w=2u l=180n
M2054 t880 t878 vdd vdd pch w=2u l=180n
CT883 t883 0 0.1f
M2055 t880 nw145 t883 0 nch w=1u l=180n
M2056 t883 t878 0 0 nch w=1u l=180n
M2057 nw146 t879 vdd vdd pch w=2u l=180n
M2058 nw146 t880 vdd vdd pch w=2u l=180n
CT884 t884 0 0.1f
M2059 nw146 t879 t884 0 nch w=1u l=180n
M2060 t884 t880 0 0 nch w=1u l=180n
Cnw146 nw146 0 2f
CT885 t885 0 0.1f
M2061 t885 nw146 vdd vdd pch w=2u l=180n
M2062 t885 nw146 0 0 nch w=1u l=180n
M2063 nq16 t885 vdd vdd pch w=2u l=180n
M2064 nq16 t885 0 0 nch w=1u l=180n
Cnq16 nq16 0 2f
CT886 t886 0 0.1f
M2065 t886 nw18 vdd vdd pch w=2u l=180n
M2066 t886 nw36 vdd vdd pch w=2u l=180n
M2067 t886 nw54 vdd vdd pch w=2u l=180n
M2068 t886 nw94 vdd vdd pch w=2u l=180n
M2069 t886 nw84 vdd vdd pch w=2u l=180n
M2070 t886 nw96 vdd vdd pch w=2u l=180n
M2071 t886 nen vdd vdd pch w=2u l=180n
CT887 t887 0 0.1f
M2072 t886 nw18 t887 0 nch w=1u l=180n
CT888 t888 0 0.1f
M2073 t887 nw36 t888 0 nch w=1u l=180n
CT889 t889 0 0.1f
M2074 t888 nw54 t889 0 nch w=1u l=180n
CT890 t890 0 0.1f
M2075 t889 nw94 t890 0 nch w=1u l=180n
CT891 t891 0 0.1f
M2076 t890 nw84 t891 0 nch w=1u l=180n
CT892 t892 0 0.1f
M2077 t891 nw96 t892 0 nch w=1u l=180n
M2078 t892 nen 0 0 nch w=1u l=180n
M2079 nw148 t886 vdd vdd pch w=2u l=180n
M2080 nw148 t886 0 0 nch w=1u l=180n
Cnw148 nw148 0 2f
CT893 t893 0 0.1f
CT894 t894 0 0.1f
CT895 t895 0 0.1f
M2081 t893 nd17 vdd vdd pch w=2u l=180n
M2082 t893 nw148 vdd vdd pch w=2u l=180n
CT896 t896 0 0.1f
M2083 t893 nd17 t896 0 nch w=1u l=180n
M2084 t896 nw148 0 0 nch w=1u l=180n
M2085 t894 nd17 vdd vdd pch w=2u l=180n
M2086 t894 t893 vdd vdd pch w=2u l=180n
CT897 t897 0 0.1f
M2087 t894 nd17 t897 0 nch w=1u l=180n
M2088 t897 t893 0 0 nch w=1u l=180n
M2089 t895 nw148 vdd vdd pch w=2u l=180n
M2090 t895 t893 vdd vdd pch w=2u l=180n
CT898 t898 0 0.1f
M2091 t895 nw148 t898 0 nch w=1u l=180n
M2092 t898 t893 0 0 nch w=1u l=180n
M2093 nw149 t894 vdd vdd pch w=2u l=180n
M2094 nw149 t895 vdd vdd pch w=2u l=180n
CT899 t899 0 0.1f
M2095 nw149 t894 t899 0 nch w=1u l=180n
M2096 t899 t895 0 0 nch w=1u l=180n
Cnw149 nw149 0 2f
CT900 t900 0 0.1f
M2097 t900 nw149 vdd vdd pch w=2u l=180n
M2098 t900 nw149 0 0 nch w=1u l=180n
M2099 nq17 t900 vdd vdd pch w=2u l=180n
M2100 nq17 t900 0 0 nch w=1u l=180n
Cnq17 nq17 0 2f
CT901 t901 0 0.1f
M2101 t901 nw91 vdd vdd pch w=2u l=180n
M2102 t901 nw92 vdd vdd pch w=2u l=180n
M2103 t901 nw93 vdd vdd pch w=2u l=180n
M2104 t901 nw69 vdd vdd pch w=2u l=180n
M2105 t901 nw84 vdd vdd pch w=2u l=180n
M2106 t901 nw96 vdd vdd pch w=2u l=180n
M2107 t901 nen vdd vdd pch w=2u l=180n
CT902 t902 0 0.1f
M2108 t901 nw91 t902 0 nch w=1u l=180n
CT903 t903 0 0.1f
M2109 t902 nw92 t903 0 nch w=1u l=180n
CT904 t904 0 0.1f
M2110 t903 nw93 t904 0 nch w=1u l=180n
CT905 t905 0 0.1f
M2111 t904 nw69 t905 0 nch w=1u l=180n
CT906 t906 0 0.1f
M2112 t905 nw84 t906 0 nch w=1u l=180n
CT907 t907 0 0.1f
M2113 t906 nw96 t907 0 nch w=1u l=180n
M2114 t907 nen 0 0 nch w=1u l=180n
M2115 nw151 t901 vdd vdd pch w=2u l=180n
M2116 nw151 t901 0 0 nch w=1u l=180n
Cnw151 nw151 0 2f
CT908 t908 0 0.1f
CT909 t909 0 0.1f
CT910 t910 0 0.1f
M2117 t908 nd18 vdd vdd pch w=2u l=180n
M2118 t908 nw151 vdd vdd pch w=2u l=180n
CT911 t911 0 0.1f
M2119 t908 nd18 t911 0 nch w=1u l=180n
M2120 t911 nw151 0 0 nch w=1u l=180n
M2121 t909 nd18 vdd vdd pch w=2u l=180n
M2122 t909 t908 vdd vdd pch w=2u l=180n
CT912 t912 0 0.1f
M2123 t909 nd18 t912 0 nch w=1u l=180n
M2124 t912 t908 0 0 nch w=1u l=180n
M2125 t910 nw151 vdd vdd pch w=2u l=180n
M2126 t910 t908 vdd vdd pch w=2u l=180n
CT913 t913 0 0.1f
M2127 t910 nw151 t913 0 nch w=1u l=180n
M2128 t913 t908 0 0 nch w=1u l=180n
M2129 nw152 t909 vdd vdd pch w=2u l=180n
M2130 nw152 t910 vdd vdd pch w=2u l=180n
CT914 t914 0 0.1f
M2131 nw152 t909 t914 0 nch w=1u l=180n
M2132 t914 t910 0 0 nch w=1u l=180n
Cnw152 nw152 0 2f
CT915 t915 0 0.1f
M2133 t915 nw152 vdd vdd pch w=2u l=180n
M2134 t915 nw152 0 0 nch w=1u l=180n
M2135 nq18 t915 vdd vdd pch w=2u l=180n
M2136 nq18 t915 0 0 nch w=1u l=180n
Cnq18 nq18 0 2f
CT916 t916 0 0.1f
M2137 t916 nw18 vdd vdd pch w=2u l=180n
M2138 t916 nw92 vdd vdd pch w=2u l=180n
M2139 t916 nw93 vdd vdd pch w=2u l=180n
M2140 t916 nw69 vdd vdd pch w=2u l=180n
M2141 t916 nw84 vdd vdd pch w=2u l=180n
M2142 t916 nw96 vdd vdd pch w=2u l=180n
M2143 t916 nen vdd vdd pch w=2u l=180n
CT917 t917 0 0.1f
M2144 t916 nw18 t917 0 nch w=1u l=180n
CT918 t918 0 0.1f
M2145 t917 nw92 t918 0 nch w=1u l=180n
CT919 t919 0 0.1f
M2146 t918 nw93 t919 0 nch w=1u l=180n
CT920 t920 0 0.1f
M2147 t919 nw69 t920 0 nch w=1u l=180n
CT921 t921 0 0.1f
M2148 t920 nw84 t921 0 nch w=1u l=180n
CT922 t922 0 0.1f
M2149 t921 nw96 t922 0 nch w=1u l=180n
M2150 t922 nen 0 0 nch w=1u l=180n
M2151 nw154 t916 vdd vdd pch w=2u l=180n
M2152 nw154 t916 0 0 nch w=1u l=180n
Cnw154 nw154 0 2f
CT923 t923 0 0.1f
CT924 t924 0 0.1f
CT925 t925 0 0.1f
M2153 t923 nd19 vdd vdd pch w=2u l=180n
M2154 t923 nw154 vdd vdd pch w=2u l=180n
CT926 t926 0 0.1f
M2155 t923 nd19 t926 0 nch w=1u l=180n
M2156 t926 nw154 0 0 nch w=1u l=180n
M2157 t924 nd19 vdd vdd pch w=2u l=180n
M2158 t924 t923 vdd vdd pch w=2u l=180n
CT927 t927 0 0.1f
M2159 t924 nd19 t927 0 nch w=1u l=180n
M2160 t927 t923 0 0 nch w=1u l=180n
M2161 t925 nw154 vdd vdd pch w=2u l=180n
M2162 t925 t923 vdd vdd pch w=2u l=180n
CT928 t928 0 0.1f
M2163 t925 nw154 t928 0 nch w=1u l=180n
M2164 t928 t923 0 0 nch w=1u l=180n
M2165 nw155 t924 vdd vdd pch w=2u l=180n
M2166 nw155 t925 vdd vdd pch w=2u l=180n
CT929 t929 0 0.1f
M2167 nw155 t924 t929 0 nch w=1u l=180n
M2168 t929 t925 0 0 nch w=1u l=180n
Cnw155 nw155 0 2f
CT930 t930 0 0.1f
M2169 t930 nw155 vdd vdd pch w=2u l=180n
M2170 t930 nw155 0 0 nch w=1u l=180n
M2171 nq19 t930 vdd vdd pch w=2u l=180n
M2172 nq19 t930 0 0 nch w=1u l=180n
Cnq19 nq19 0 2f
CT931 t931 0 0.1f
M2173 t931 nw91 vdd vdd pch w=2u l=180n
M2174 t931 nw36 vdd vdd pch w=2u l=180n
M2175 t931 nw93 vdd vdd pch w=2u l=180n
M2176 t931 nw69 vdd vdd pch w=2u l=180n
M2177 t931 nw84 vdd vdd pch w=2u l=180n
M2178 t931 nw96 vdd vdd pch w=2u l=180n
M2179 t931 nen vdd vdd pch w=2u l=180n
CT932 t932 0 0.1f
M2180 t931 nw91 t932 0 nch w=1u l=180n
CT933 t933 0 0.1f
M2181 t932 nw36 t933 0 nch w=1u l=180n
CT934 t934 0 0.1f
M2182 t933 nw93 t934 0 nch w=1u l=180n
CT935 t935 0 0.1f
M2183 t934 nw69 t935 0 nch w=1u l=180n
CT936 t936 0 0.1f
M2184 t935 nw84 t936 0 nch w=1u l=180n
CT937 t937 0 0.1f
M2185 t936 nw96 t937 0 nch w=1u l=180n
M2186 t937 nen 0 0 nch w=1u l=180n
M2187 nw157 t931 vdd vdd pch w=2u l=180n
M2188 nw157 t931 0 0 nch w=1u l=180n
Cnw157 nw157 0 2f
CT938 t938 0 0.1f
CT939 t939 0 0.1f
CT940 t940 0 0.1f
M2189 t938 nd20 vdd vdd pch w=2u l=180n
M2190 t938 nw157 vdd vdd pch w=2u l=180n
CT941 t941 0 0.1f
M2191 t938 nd20 t941 0 nch w=1u l=180n
M2192 t941 nw157 0 0 nch w=1u l=180n
M2193 t939 nd20 vdd vdd pch w=2u l=180n
M2194 t939 t938 vdd vdd pch w=2u l=180n
CT942 t942 0 0.1f
M2195 t939 nd20 t942 0 nch w=1u l=180n
M2196 t942 t938 0 0 nch w=1u l=180n
M2197 t940 nw157 vdd vdd pch w=2u l=180n
M2198 t940 t938 vdd vdd pch w=2u l=180n
CT943 t943 0 0.1f
M2199 t940 nw157 t943 0 nch w=1u l=180n
M2200 t943 t938 0 0 nch w=1u l=180n
M2201 nw158 t939 vdd vdd pch w=2u l=180n
M2202 nw158 t940 vdd vdd pch w=2u l=180n
CT944 t944 0 0.1f
M2203 nw158 t939 t944 0 nch w=1u l=180n
M2204 t944 t940 0 0 nch w=1u l=180n
Cnw158 nw158 0 2f
CT945 t945 0 0.1f
M2205 t945 nw158 vdd vdd pch w=2u l=180n
M2206 t945 nw158 0 0 nch w=1u l=180n
M2207 nq20 t945 vdd vdd pch w=2u l=180n
M2208 nq20 t945 0 0 nch w=1u l=180n
Cnq20 nq20 0 2f
CT946 t946 0 0.1f
M2209 t946 nw18 vdd vdd pch w=2u l=180n
M2210 t946 nw36 vdd vdd pch w=2u l=180n
M2211 t946 nw93 vdd vdd pch w=2u l=180n
M2212 t946 nw69 vdd vdd pch w=2u l=180n
M2213 t946 nw84 vdd vdd pch w=2u l=180n
M2214 t946 nw96 vdd vdd pch w=2u l=180n
M2215 t946 nen vdd vdd pch w=2u l=180n
CT947 t947 0 0.1f
M2216 t946 nw18 t947 0 nch w=1u l=180n
CT948 t948 0 0.1f
M2217 t947 nw36 t948 0 nch w=1u l=180n
CT949 t949 0 0.1f
M2218 t948 nw93 t949 0 nch w=1u l=180n
CT950 t950 0 0.1f
M2219 t949 nw69 t950 0 nch w=1u l=180n
CT951 t951 0 0.1f
M2220 t950 nw84 t951 0 nch w=1u l=180n
CT952 t952 0 0.1f
M2221 t951 nw96 t952 0 nch w=1u l=180n
M2222 t952 nen 0 0 nch w=1u l=180n
M2223 nw160 t946 vdd vdd pch w=2u l=180n
M2224 nw160 t946 0 0 nch w=1u l=180n
Cnw160 nw160 0 2f
CT953 t953 0 0.1f
CT954 t954 0 0.1f
CT955 t955 0 0.1f
M2225 t953 nd21 vdd vdd pch w=2u l=180n
M2226 t953 nw160 vdd vdd pch w=2u l=180n
CT956 t956 0 0.1f
M2227 t953 nd21 t956 0 nch w=1u l=180n
M2228 t956 nw160 0 0 nch w=1u l=180n
M2229 t954 nd21 vdd vdd pch w=2u l=180n
M2230 t954 t953 vdd vdd pch w=2u l=180n
CT957 t957 0 0.1f
M2231 t954 nd21 t957 0 nch w=1u l=180n
M2232 t957 t953 0 0 nch w=1u l=180n
M2233 t955 nw160 vdd vdd pch w=2u l=180n
M2234 t955 t953 vdd vdd pch w=2u l=180n
CT958 t958 0 0.1f
M2235 t955 nw160 t958 0 nch w=1u l=180n
M2236 t958 t953 0 0 nch w=1u l=180n
M2237 nw161 t954 vdd vdd pch w=2u l=180n
M2238 nw161 t955 vdd vdd pch w=2u l=180n
CT959 t959 0 0.1f
M2239 nw161 t954 t959 0 nch w=1u l=180n
M2240 t959 t955 0 0 nch w=1u l=180n
Cnw161 nw161 0 2f
CT960 t960 0 0.1f
M2241 t960 nw161 vdd vdd pch w=2u l=180n
M2242 t960 nw161 0 0 nch w=1u l=180n
M2243 nq21 t960 vdd vdd pch w=2u l=180n
M2244 nq21 t960 0 0 nch w=1u l=180n
Cnq21 nq21 0 2f
CT961 t961 0 0.1f
M2245 t961 nw91 vdd vdd pch w=2u l=180n
M2246 t961 nw92 vdd vdd pch w=2u l=180n
M2247 t961 nw54 vdd vdd pch w=2u l=180n
M2248 t961 nw69 vdd vdd pch w=2u l=180n
M2249 t961 nw84 vdd vdd pch w=2u l=180n
M2250 t961 nw96 vdd vdd pch w=2u l=180n
M2251 t961 nen vdd vdd pch w=2u l=180n
CT962 t962 0 0.1f
M2252 t961 nw91 t962 0 nch w=1u l=180n
CT963 t963 0 0.1f
M2253 t962 nw92 t963 0 nch w=1u l=180n
CT964 t964 0 0.1f
M2254 t963 nw54 t964 0 nch w=1u l=180n
CT965 t965 0 0.1f
M2255 t964 nw69 t965 0 nch w=1u l=180n
CT966 t966 0 0.1f
M2256 t965 nw84 t966 0 nch w=1u l=180n
CT967 t967 0 0.1f
M2257 t966 nw96 t967 0 nch w=1u l=180n
M2258 t967 nen 0 0 nch w=1u l=180n
M2259 nw163 t961 vdd vdd pch w=2u l=180n
M2260 nw163 t961 0 0 nch w=1u l=180n
Cnw163 nw163 0 2f
CT968 t968 0 0.1f
CT969 t969 0 0.1f
CT970 t970 0 0.1f
M2261 t968 nd22 vdd vdd pch w=2u l=180n
M2262 t968 nw163 vdd vdd pch w=2u l=180n
CT971 t971 0 0.1f
M2263 t968 nd22 t971 0 nch w=1u l=180n
M2264 t971 nw163 0 0 nch w=1u l=180n
M2265 t969 nd22 vdd vdd pch w=2u l=180n
M2266 t969 t968 vdd vdd pch w=2u l=180n
CT972 t972 0 0.1f
M2267 t969 nd22 t972 0 nch w=1u l=180n
M2268 t972 t968 0 0 nch w=1u l=180n
M2269 t970 nw163 vdd vdd pch w=2u l=180n
M2270 t970 t968 vdd vdd pch w=2u l=180n
CT973 t973 0 0.1f
M2271 t970 nw163 t973 0 nch w=1u l=180n
M2272 t973 t968 0 0 nch w=1u l=180n
M2273 nw164 t969 vdd vdd pch w=2u l=180n
M2274 nw164 t970 vdd vdd pch w=2u l=180n
CT974 t974 0 0.1f
M2275 nw164 t969 t974 0 nch w=1u l=180n
M2276 t974 t970 0 0 nch w=1u l=180n
Cnw164 nw164 0 2f
CT975 t975 0 0.1f
M2277 t975 nw164 vdd vdd pch w=2u l=180n
M2278 t975 nw164 0 0 nch w=1u l=180n
M2279 nq22 t975 vdd vdd pch w=2u l=180n
M2280 nq22 t975 0 0 nch w=1u l=180n
Cnq22 nq22 0 2f
CT976 t976 0 0.1f
M2281 t976 nw18 vdd vdd pch w=2u l=180n
M2282 t976 nw92 vdd vdd pch w=2u l=180n
M2283 t976 nw54 vdd vdd pch w=2u l=180n
M2284 t976 nw69 vdd vdd pch w=2u l=180n
M2285 t976 nw84 vdd vdd pch w=2u l=180n
M2286 t976 nw96 vdd vdd pch w=2u l=180n
M2287 t976 nen vdd vdd pch w=2u l=180n
CT977 t977 0 0.1f
M2288 t976 nw18 t977 0 nch w=1u l=180n
CT978 t978 0 0.1f
M2289 t977 nw92 t978 0 nch w=1u l=180n
CT979 t979 0 0.1f
M2290 t978 nw54 t979 0 nch w=1u l=180n
CT980 t980 0 0.1f
M2291 t979 nw69 t980 0 nch w=1u l=180n
CT981 t981 0 0.1f
M2292 t980 nw84 t981 0 nch w=1u l=180n
CT982 t982 0 0.1f
M2293 t981 nw96 t982 0 nch w=1u l=180n
M2294 t982 nen 0 0 nch w=1u l=180n
M2295 nw166 t976 vdd vdd pch w=2u l=180n
M2296 nw166 t976 0 0 nch w=1u l=180n
Cnw166 nw166 0 2f
CT983 t983 0 0.1f
CT984 t984 0 0.1f
CT985 t985 0 0.1f
M2297 t983 nd23 vdd vdd pch w=2u l=180n
M2298 t983 nw166 vdd vdd pch w=2u l=180n
CT986 t986 0 0.1f
M2299 t983 nd23 t986 0 nch w=1u l=180n
M2300 t986 nw166 0 0 nch w=1u l=180n
M2301 t984 nd23 vdd vdd pch w=2u l=180n
M2302 t984 t983 vdd vdd pch w=2u l=180n
CT987 t987 0 0.1f
M2303 t984 nd23 t987 0 nch w=1u l=180n
M2304 t987 t983 0 0 nch w=1u l=180n
M2305 t985 nw166 vdd vdd pch w=2u l=180n
M2306 t985 t983 vdd vdd pch w=2u l=180n
CT988 t988 0 0.1f
M2307 t985 nw166 t988 0 nch w=1u l=180n
M2308 t988 t983 0 0 nch w=1u l=180n
M2309 nw167 t984 vdd vdd pch w=2u l=180n
M2310 nw167 t985 vdd vdd pch w=2u l=180n
CT989 t989 0 0.1f
M2311 nw167 t984 t989 0 nch w=1u l=180n
M2312 t989 t985 0 0 nch w=1u l=180n
Cnw167 nw167 0 2f
CT990 t990 0 0.1f
M2313 t990 nw167 vdd vdd pch w=2u l=180n
M2314 t990 nw167 0 0 nch w=1u l=180n
M2315 nq23 t990 vdd vdd pch w=2u l=180n
M2316 nq23 t990 0 0 nch w=1u l=180n
Cnq23 nq23 0 2f
CT991 t991 0 0.1f
M2317 t991 nw91 vdd vdd pch w=2u l=180n
M2318 t991 nw36 vdd vdd pch w=2u l=180n
M2319 t991 nw54 vdd vdd pch w=2u l=180n
M2320 t991 nw69 vdd vdd pch w=2u l=180n
M2321 t991 nw84 vdd vdd pch w=2u l=180n
M2322 t991 nw96 vdd vdd pch w=2u l=180n
M2323 t991 nen vdd vdd pch w=2u l=180n
CT992 t992 0 0.1f
M2324 t991 nw91 t992 0 nch w=1u l=180n
CT993 t993 0 0.1f
M2325 t992 nw36 t993 0 nch w=1u l=180n
CT994 t994 0 0.1f
M2326 t993 nw54 t994 0 nch w=1u l=180n
CT995 t995 0 0.1f
M2327 t994 nw69 t995 0 nch w=1u l=180n
CT996 t996 0 0.1f
M2328 t995 nw84 t996 0 nch w=1u l=180n
CT997 t997 0 0.1f
M2329 t996 nw96 t997 0 nch w=1u l=180n
M2330 t997 nen 0 0 nch w=1u l=180n
M2331 nw169 t991 vdd vdd pch w=2u l=180n
M2332 nw169 t991 0 0 nch w=1u l=180n
Cnw169 nw169 0 2f
CT998 t998 0 0.1f
CT999 t999 0 0.1f
CT1000 t1000 0 0.1f
M2333 t998 nd24 vdd vdd pch w=2u l=180n
M2334 t998 nw169 vdd vdd pch w=2u l=180n
CT1001 t1001 0 0.1f
M2335 t998 nd24 t1001 0 nch w=1u l=180n
M2336 t1001 nw169 0 0 nch w=1u l=180n
M2337 t999 nd24 vdd vdd pch w=2u l=180n
M2338 t999 t998 vdd vdd pch w=2u l=180n
CT1002 t1002 0 0.1f
M2339 t999 nd24 t1002 0 nch w=1u l=180n
M2340 t1002 t998 0 0 nch w=1u l=180n
M2341 t1000 nw169 vdd vdd pch w=2u l=180n
M2342 t1000 t998 vdd vdd pch w=2u l=180n
CT1003 t1003 0 0.1f
M2343 t1000 nw169 t1003 0 nch w=1u l=180n
M2344 t1003 t998 0 0 nch w=1u l=180n
M2345 nw170 t999 vdd vdd pch w=2u l=180n
M2346 nw170 t1000 vdd vdd pch w=2u l=180n
CT1004 t1004 0 0.1f
M2347 nw170 t999 t1004 0 nch w=1u l=180n
M2348 t1004 t1000 0 0 nch w=1u l=180n
Cnw170 nw170 0 2f
CT1005 t1005 0 0.1f
M2349 t1005 nw170 vdd vdd pch w=2u l=180n
M2350 t1005 nw170 0 0 nch w=1u l=180n
M2351 nq24 t1005 vdd vdd pch w=2u l=180n
M2352 nq24 t1005 0 0 nch w=1u l=180n
Cnq24 nq24 0 2f
CT1006 t1006 0 0.1f
M2353 t1006 nw18 vdd vdd pch w=2u l=180n
M2354 t1006 nw36 vdd vdd pch w=2u l=180n
M2355 t1006 nw54 vdd vdd pch w=2u l=180n
M2356 t1006 nw69 vdd vdd pch w=2u l=180n
M2357 t1006 nw84 vdd vdd pch w=2u l=180n
M2358 t1006 nw96 vdd vdd pch w=2u l=180n
M2359 t1006 nen vdd vdd pch w=2u l=180n
CT1007 t1007 0 0.1f
M2360 t1006 nw18 t1007 0 nch w=1u l=180n
CT1008 t1008 0 0.1f
M2361 t1007 nw36 t1008 0 nch w=1u l=180n
CT1009 t1009 0 0.1f
M2362 t1008 nw54 t1009 0 nch w=1u l=180n
CT1010 t1010 0 0.1f
M2363 t1009 nw69 t1010 0 nch w=1u l=180n
CT1011 t1011 0 0.1f
M2364 t1010 nw84 t1011 0 nch w=1u l=180n
CT1012 t1012 0 0.1f
M2365 t1011 nw96 t1012 0 nch w=1u l=180n
M2366 t1012 nen 0 0 nch w=1u l=180n
M2367 nw172 t1006 vdd vdd pch w=2u l=180n
M2368 nw172 t1006 0 0 nch w=1u l=180n
Cnw172 nw172 0 2f
CT1013 t1013 0 0.1f
CT1014 t1014 0 0.1f
CT1015 t1015 0 0.1f
M2369 t1013 nd25 vdd vdd pch w=2u l=180n
M2370 t1013 nw172 vdd vdd pch w=2u l=180n
CT1016 t1016 0 0.1f
M2371 t1013 nd25 t1016 0 nch w=1u l=180n
M2372 t1016 nw172 0 0 nch w=1u l=180n
M2373 t1014 nd25 vdd vdd pch w=2u l=180n
M2374 t1014 t1013 vdd vdd pch w=2u l=180n
CT1017 t1017 0 0.1f
M2375 t1014 nd25 t1017 0 nch w=1u l=180n
M2376 t1017 t1013 0 0 nch w=1u l=180n
M2377 t1015 nw172 vdd vdd pch w=2u l=180n
M2378 t1015 t1013 vdd vdd pch w=2u l=180n
CT1018 t1018 0 0.1f
M2379 t1015 nw172 t1018 0 nch w=1u l=180n
M2380 t1018 t1013 0 0 nch w=1u l=180n
M2381 nw173 t1014 vdd vdd pch w=2u l=180n
M2382 nw173 t1015 vdd vdd pch w=2u l=180n
CT1019 t1019 0 0.1f
M2383 nw173 t1014 t1019 0 nch w=1u l=180n
M2384 t1019 t1015 0 0 nch w=1u l=180n
Cnw173 nw173 0 2f
CT1020 t1020 0 0.1f
M2385 t1020 nw173 vdd vdd pch w=2u l=180n
M2386 t1020 nw173 0 0 nch w=1u l=180n
M2387 nq25 t1020 vdd vdd pch w=2u l=180n
M2388 nq25 t1020 0 0 nch w=1u l=180n
Cnq25 nq25 0 2f
CT1021 t1021 0 0.1f
M2389 t1021 nw18 vdd vdd pch w=2u l=180n
M2390 t1021 nw92 vdd vdd pch w=2u l=180n
M2391 t1021 nw93 vdd vdd pch w=2u l=180n
M2392 t1021 nw94 vdd vdd pch w=2u l=180n
M2393 t1021 nw95 vdd vdd pch w=2u l=180n
M2394 t1021 nw90 vdd vdd pch w=2u l=180n
M2395 t1021 nen vdd vdd pch w=2u l=180n
CT1022 t1022 0 0.1f
M2396 t1021 nw18 t1022 0 nch w=1u l=180n
CT1023 t1023 0 0.1f
M2397 t1022 nw92 t1023 0 nch w=1u l=180n
CT1024 t1024 0 0.1f
M2398 t1023 nw93 t1024 0 nch w=1u l=180n
CT1025 t1025 0 0.1f
M2399 t1024 nw94 t1025 0 nch w=1u l=180n
CT1026 t1026 0 0.1f
M2400 t1025 nw95 t1026 0 nch w=1u l=180n
CT1027 t1027 0 0.1f
M2401 t1026 nw90 t1027 0 nch w=1u l=180n
M2402 t1027 nen 0 0 nch w=1u l=180n
M2403 nw175 t1021 vdd vdd pch w=2u l=180n
M2404 nw175 t1021 0 0 nch w=1u l=180n
Cnw175 nw175 0 2f
CT1028 t1028 0 0.1f
CT1029 t1029 0 0.1f
CT1030 t1030 0 0.1f
M2405 t1028 nd26 vdd vdd pch w=2u l=180n
M2406 t1028 nw175 vdd vdd pch w=2u l=180n
CT1031 t1031 0 0.1f
M2407 t1028 nd26 t1031 0 nch w=1u l=180n
M2408 t1031 nw175 0 0 nch w=1u l=180n
M2409 t1029 nd26 vdd vdd pch w=2u l=180n
M2410 t1029 t1028 vdd vdd pch w=2u l=180n
CT1032 t1032 0 0.1f
M2411 t1029 nd26 t1032 0 nch w=1u l=180n
M2412 t1032 t1028 0 0 nch w=1u l=180n
M2413 t1030 nw175 vdd vdd pch w=2u l=180n
M2414 t1030 t1028 vdd vdd pch w=2u l=180n
CT1033 t1033 0 0.1f
M2415 t1030 nw175 t1033 0 nch w=1u l=180n
M2416 t1033 t1028 0 0 nch w=1u l=180n
M2417 nw176 t1029 vdd vdd pch w=2u l=180n
M2418 nw176 t1030 vdd vdd pch w=2u l=180n
CT1034 t1034 0 0.1f
M2419 nw176 t1029 t1034 0 nch w=1u l=180n
M2420 t1034 t1030 0 0 nch w=1u l=180n
Cnw176 nw176 0 2f
CT1035 t1035 0 0.1f
M2421 t1035 nw176 vdd vdd pch w=2u l=180n
M2422 t1035 nw176 0 0 nch w=1u l=180n
M2423 nq26 t1035 vdd vdd pch w=2u l=180n
M2424 nq26 t1035 0 0 nch w=1u l=180n
Cnq26 nq26 0 2f
CT1036 t1036 0 0.1f
M2425 t1036 nw91 vdd vdd pch w=2u l=180n
M2426 t1036 nw36 vdd vdd pch w=2u l=180n
M2427 t1036 nw93 vdd vdd pch w=2u l=180n
M2428 t1036 nw94 vdd vdd pch w=2u l=180n
M2429 t1036 nw95 vdd vdd pch w=2u l=180n
M2430 t1036 nw90 vdd vdd pch w=2u l=180n
M2431 t1036 nen vdd vdd pch w=2u l=180n
CT1037 t1037 0 0.1f
M2432 t1036 nw91 t1037 0 nch w=1u l=180n
CT1038 t1038 0 0.1f
M2433 t1037 nw36 t1038 0 nch w=1u l=180n
CT1039 t1039 0 0.1f
M2434 t1038 nw93 t1039 0 nch w=1u l=180n
CT1040 t1040 0 0.1f
M2435 t1039 nw94 t1040 0 nch w=1u l=180n
CT1041 t1041 0 0.1f
M2436 t1040 nw95 t1041 0 nch w=1u l=180n
CT1042 t1042 0 0.1f
M2437 t1041 nw90 t1042 0 nch w=1u l=180n
M2438 t1042 nen 0 0 nch w=1u l=180n
M2439 nw178 t1036 vdd vdd pch w=2u l=180n
M2440 nw178 t1036 0 0 nch w=1u l=180n
Cnw178 nw178 0 2f
CT1043 t1043 0 0.1f
CT1044 t1044 0 0.1f
CT1045 t1045 0 0.1f
M2441 t1043 nd27 vdd vdd pch w=2u l=180n
M2442 t1043 nw178 vdd vdd pch w=2u l=180n
CT1046 t1046 0 0.1f
M2443 t1043 nd27 t1046 0 nch w=1u l=180n
M2444 t1046 nw178 0 0 nch w=1u l=180n
M2445 t1044 nd27 vdd vdd pch w=2u l=180n
M2446 t1044 t1043 vdd vdd pch w=2u l=180n
CT1047 t1047 0 0.1f
M2447 t1044 nd27 t1047 0 nch w=1u l=180n
M2448 t1047 t1043 0 0 nch w=1u l=180n
M2449 t1045 nw178 vdd vdd pch w=2u l=180n
M2450 t1045 t1043 vdd vdd pch w=2u l=180n
CT1048 t1048 0 0.1f
M2451 t1045 nw178 t1048 0 nch w=1u l=180n
M2452 t1048 t1043 0 0 nch w=1u l=180n
M2453 nw179 t1044 vdd vdd pch w=2u l=180n
M2454 nw179 t1045 vdd vdd pch w=2u l=180n
CT1049 t1049 0 0.1f
M2455 nw179 t1044 t1049 0 nch w=1u l=180n
M2456 t1049 t1045 0 0 nch w=1u l=180n
Cnw179 nw179 0 2f
CT1050 t1050 0 0.1f
M2457 t1050 nw179 vdd vdd pch w=2u l=180n
M2458 t1050 nw179 0 0 nch w=1u l=180n
M2459 nq27 t1050 vdd vdd pch w=2u l=180n
M2460 nq27 t1050 0 0 nch w=1u l=180n
Cnq27 nq27 0 2f
CT1051 t1051 0 0.1f
M2461 t1051 nw18 vdd vdd pch w=2u l=180n
M2462 t1051 nw36 vdd vdd pch w=2u l=180n
M2463 t1051 nw93 vdd vdd pch w=2u l=180n
M2464 t1051 nw94 vdd vdd pch w=2u l=180n
M2465 t1051 nw95 vdd vdd pch w=2u l=180n
M2466 t1051 nw90 vdd vdd pch w=2u l=180n
M2467 t1051 nen vdd vdd pch w=2u l=180n
CT1052 t1052 0 0.1f
M2468 t1051 nw18 t1052 0 nch w=1u l=180n
CT1053 t1053 0 0.1f
M2469 t1052 nw36 t1053 0 nch w=1u l=180n
CT1054 t1054 0 0.1f
M2470 t1053 nw93 t1054 0 nch w=1u l=180n
CT1055 t1055 0 0.1f
M2471 t1054 nw94 t1055 0 nch w=1u l=180n
CT1056 t1056 0 0.1f
M2472 t1055 nw95 t1056 0 nch w=1u l=180n
CT1057 t1057 0 0.1f
M2473 t1056 nw90 t1057 0 nch w=1u l=180n
M2474 t1057 nen 0 0 nch w=1u l=180n
M2475 nw181 t1051 vdd vdd pch w=2u l=180n
M2476 nw181 t1051 0 0 nch w=1u l=180n
Cnw181 nw181 0 2f
CT1058 t1058 0 0.1f
CT1059 t1059 0 0.1f
CT1060 t1060 0 0.1f
M2477 t1058 nd28 vdd vdd pch w=2u l=180n
M2478 t1058 nw181 vdd vdd pch w=2u l=180n
CT1061 t1061 0 0.1f
M2479 t1058 nd28 t1061 0 nch w=1u l=180n
M2480 t1061 nw181 0 0 nch w=1u l=180n
M2481 t1059 nd28 vdd vdd pch w=2u l=180n
M2482 t1059 t1058 vdd vdd pch w=2u l=180n
CT1062 t1062 0 0.1f
M2483 t1059 nd28 t1062 0 nch w=1u l=180n
M2484 t1062 t1058 0 0 nch w=1u l=180n
M2485 t1060 nw181 vdd vdd pch w=2u l=180n
M2486 t1060 t1058 vdd vdd pch w=2u l=180n
CT1063 t1063 0 0.1f
M2487 t1060 nw181 t1063 0 nch w=1u l=180n
M2488 t1063 t1058 0 0 nch w=1u l=180n
M2489 nw182 t1059 vdd vdd pch w=2u l=180n
M2490 nw182 t1060 vdd vdd pch w=2u l=180n
CT1064 t1064 0 0.1f
M2491 nw182 t1059 t1064 0 nch w=1u l=180n
M2492 t1064 t1060 0 0 nch w=1u l=180n
Cnw182 nw182 0 2f
CT1065 t1065 0 0.1f
M2493 t1065 nw182 vdd vdd pch w=2u l=180n
M2494 t1065 nw182 0 0 nch w=1u l=180n
M2495 nq28 t1065 vdd vdd pch w=2u l=180n
M2496 nq28 t1065 0 0 nch w=1u l=180n
Cnq28 nq28 0 2f
CT1066 t1066 0 0.1f
M2497 t1066 nw91 vdd vdd pch w=2u l=180n
M2498 t1066 nw92 vdd vdd pch w=2u l=180n
M2499 t1066 nw54 vdd vdd pch w=2u l=180n
M2500 t1066 nw94 vdd vdd pch w=2u l=180n
M2501 t1066 nw95 vdd vdd pch w=2u l=180n
M2502 t1066 nw90 vdd vdd pch w=2u l=180n
M2503 t1066 nen vdd vdd pch w=2u l=180n
CT1067 t1067 0 0.1f
M2504 t1066 nw91 t1067 0 nch w=1u l=180n
CT1068 t1068 0 0.1f
M2505 t1067 nw92 t1068 0 nch w=1u l=180n
CT1069 t1069 0 0.1f
M2506 t1068 nw54 t1069 0 nch w=1u l=180n
CT1070 t1070 0 0.1f
M2507 t1069 nw94 t1070 0 nch w=1u l=180n
CT1071 t1071 0 0.1f
M2508 t1070 nw95 t1071 0 nch w=1u l=180n
CT1072 t1072 0 0.1f
M2509 t1071 nw90 t1072 0 nch w=1u l=180n
M2510 t1072 nen 0 0 nch w=1u l=180n
M2511 nw184 t1066 vdd vdd pch w=2u l=180n
M2512 nw184 t1066 0 0 nch w=1u l=180n
Cnw184 nw184 0 2f
CT1073 t1073 0 0.1f
CT1074 t1074 0 0.1f
CT1075 t1075 0 0.1f
M2513 t1073 nd29 vdd vdd pch w=2u l=180n
M2514 t1073 nw184 vdd vdd pch w=2u l=180n
CT1076 t1076 0 0.1f
M2515 t1073 nd29 t1076 0 nch w=1u l=180n
M2516 t1076 nw184 0 0 nch w=1u l=180n
M2517 t1074 nd29 vdd vdd pch w=2u l=180n
M2518 t1074 t1073 vdd vdd pch w=2u l=180n
CT1077 t1077 0 0.1f
M2519 t1074 nd29 t1077 0 nch w=1u l=180n
M2520 t1077 t1073 0 0 nch w=1u l=180n
M2521 t1075 nw184 vdd vdd pch w=2u l=180n
M2522 t1075 t1073 vdd vdd pch w=2u l=180n
CT1078 t1078 0 0.1f
M2523 t1075 nw184 t1078 0 nch w=1u l=180n
M2524 t1078 t1073 0 0 nch w=1u l=180n
M2525 nw185 t1074 vdd vdd pch w=2u l=180n
M2526 nw185 t1075 vdd vdd pch w=2u l=180n
CT1079 t1079 0 0.1f
M2527 nw185 t1074 t1079 0 nch w=1u l=180n
M2528 t1079 t1075 0 0 nch w=1u l=180n
Cnw185 nw185 0 2f
CT1080 t1080 0 0.1f
M2529 t1080 nw185 vdd vdd pch w=2u l=180n
M2530 t1080 nw185 0 0 nch w=1u l=180n
M2531 nq29 t1080 vdd vdd pch w=2u l=180n
M2532 nq29 t1080 0 0 nch w=1u l=180n
Cnq29 nq29 0 2f
CT1081 t1081 0 0.1f
M2533 t1081 nw18 vdd vdd pch w=2u l=180n
M2534 t1081 nw92 vdd vdd pch w=2u l=180n
M2535 t1081 nw54 vdd vdd pch w=2u l=180n
M2536 t1081 nw94 vdd vdd pch w=2u l=180n
M2537 t1081 nw95 vdd vdd pch w=2u l=180n
M2538 t1081 nw90 vdd vdd pch w=2u l=180n
M2539 t1081 nen vdd vdd pch w=2u l=180n
CT1082 t1082 0 0.1f
M2540 t1081 nw18 t1082 0 nch w=1u l=180n
CT1083 t1083 0 0.1f
M2541 t1082 nw92 t1083 0 nch w=1u l=180n
CT1084 t1084 0 0.1f
M2542 t1083 nw54 t1084 0 nch w=1u l=180n
CT1085 t1085 0 0.1f
M2543 t1084 nw94 t1085 0 nch w=1u l=180n
CT1086 t1086 0 0.1f
M2544 t1085 nw95 t1086 0 nch w=1u l=180n
CT1087 t1087 0 0.1f
M2545 t1086 nw90 t1087 0 nch w=1u l=180n
M2546 t1087 nen 0 0 nch w=1u l=180n
M2547 nw187 t1081 vdd vdd pch w=2u l=180n
M2548 nw187 t1081 0 0 nch w=1u l=180n
Cnw187 nw187 0 2f
CT1088 t1088 0 0.1f
CT1089 t1089 0 0.1f
CT1090 t1090 0 0.1f
M2549 t1088 nd30 vdd vdd pch w=2u l=180n
M2550 t1088 nw187 vdd vdd pch w=2u l=180n
CT1091 t1091 0 0.1f
M2551 t1088 nd30 t1091 0 nch w=1u l=180n
M2552 t1091 nw187 0 0 nch w=1u l=180n
M2553 t1089 nd30 vdd vdd pch w=2u l=180n
M2554 t1089 t1088 vdd vdd pch w=2u l=180n
CT1092 t1092 0 0.1f
M2555 t1089 nd30 t1092 0 nch w=1u l=180n
M2556 t1092 t1088 0 0 nch w=1u l=180n
M2557 t1090 nw187 vdd vdd pch w=2u l=180n
M2558 t1090 t1088 vdd vdd pch w=2u l=180n
CT1093 t1093 0 0.1f
M2559 t1090 nw187 t1093 0 nch w=1u l=180n
M2560 t1093 t1088 0 0 nch w=1u l=180n
M2561 nw188 t1089 vdd vdd pch w=2u l=180n
M2562 nw188 t1090 vdd vdd pch w=2u l=180n
CT1094 t1094 0 0.1f
M2563 nw188 t1089 t1094 0 nch w=1u l=180n
M2564 t1094 t1090 0 0 nch w=1u l=180n
Cnw188 nw188 0 2f
CT1095 t1095 0 0.1f
M2565 t1095 nw188 vdd vdd pch w=2u l=180n
M2566 t1095 nw188 0 0 nch w=1u l=180n
M2567 nq30 t1095 vdd vdd pch w=2u l=180n
M2568 nq30 t1095 0 0 nch w=1u l=180n
Cnq30 nq30 0 2f
CT1096 t1096 0 0.1f
M2569 t1096 nw91 vdd vdd pch w=2u l=180n
M2570 t1096 nw36 vdd vdd pch w=2u l=180n
M2571 t1096 nw54 vdd vdd pch w=2u l=180n
M2572 t1096 nw94 vdd vdd pch w=2u l=180n
M2573 t1096 nw95 vdd vdd pch w=2u l=180n
M2574 t1096 nw90 vdd vdd pch w=2u l=180n
M2575 t1096 nen vdd vdd pch w=2u l=180n
CT1097 t1097 0 0.1f
M2576 t1096 nw91 t1097 0 nch w=1u l=180n
CT1098 t1098 0 0.1f
M2577 t1097 nw36 t1098 0 nch w=1u l=180n
CT1099 t1099 0 0.1f
M2578 t1098 nw54 t1099 0 nch w=1u l=180n
CT1100 t1100 0 0.1f
M2579 t1099 nw94 t1100 0 nch w=1u l=180n
CT1101 t1101 0 0.1f
M2580 t1100 nw95 t1101 0 nch w=1u l=180n
CT1102 t1102 0 0.1f
M2581 t1101 nw90 t1102 0 nch w=1u l=180n
M2582 t1102 nen 0 0 nch w=1u l=180n
M2583 nw190 t1096 vdd vdd pch w=2u l=180n
M2584 nw190 t1096 0 0 nch w=1u l=180n
Cnw190 nw190 0 2f
CT1103 t1103 0 0.1f
CT1104 t1104 0 0.1f
CT1105 t1105 0 0.1f
M2585 t1103 nd31 vdd vdd pch w=2u l=180n
M2586 t1103 nw190 vdd vdd pch w=2u l=180n
CT1106 t1106 0 0.1f
M2587 t1103 nd31 t1106 0 nch w=1u l=180n
M2588 t1106 nw190 0 0 nch w=1u l=180n
M2589 t1104 nd31 vdd vdd pch w=2u l=180n
M2590 t1104 t1103 vdd vdd pch w=2u l=180n
CT1107 t1107 0 0.1f
M2591 t1104 nd31 t1107 0 nch w=1u l=180n
M2592 t1107 t1103 0 0 nch w=1u l=180n
M2593 t1105 nw190 vdd vdd pch w=2u l=180n
M2594 t1105 t1103 vdd vdd pch w=2u l=180n
CT1108 t1108 0 0.1f
M2595 t1105 nw190 t1108 0 nch w=1u l=180n
M2596 t1108 t1103 0 0 nch w=1u l=180n
M2597 nw191 t1104 vdd vdd pch w=2u l=180n
M2598 nw191 t1105 vdd vdd pch w=2u l=180n
CT1109 t1109 0 0.1f
M2599 nw191 t1104 t1109 0 nch w=1u l=180n
M2600 t1109 t1105 0 0 nch w=1u l=180n
Cnw191 nw191 0 2f
CT1110 t1110 0 0.1f
M2601 t1110 nw191 vdd vdd pch w=2u l=180n
M2602 t1110 nw191 0 0 nch w=1u l=180n
M2603 nq31 t1110 vdd vdd pch w=2u l=180n
M2604 nq31 t1110 0 0 nch w=1u l=180n
Cnq31 nq31 0 2f
.model nch NMOS (vto=0.45 kp=200u lambda=0.05)
.model pch PMOS (vto=-0.45 kp=100u lambda=0.05)
* outputs: nq0 nq1 nq2 nq3 nq4 nq5 nq6 nq7 nq8 nq9 nq10 nq11 nq12 nq13 nq14 nq15 nq16 nq17 nq18 nq19 nq20 nq21 nq22 nq23 nq24 nq25 nq26 nq27 nq28 nq29 nq30 nq31
.end
