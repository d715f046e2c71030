* s382 (s382: traffic-light controller, 21 flip-flops): 190 gates, 1502 transistors
VDD vdd 0 DC 1.8
VIN0 ni0 0 PULSE(0 1.8 5e-10 20p 20p 1e-09 2e-09)
VIN1 ni1 0 PULSE(0 1.8 1e-09 20p 20p 2e-09 4e-09)
VIN2 ni2 0 PULSE(0 1.8 2e-09 20p 20p 4e-09 8e-09)
VIN3 ni3 0 PULSE(0 1.8 4e-09 20p 20p 8e-09 1.6e-08)
VIN4 ni4 0 PULSE(0 1.8 8e-09 20p 20p 1.6e-08 3.2e-08)
VIN5 ni5 0 PULSE(0 1.8 1.6e-08 20p 20p 3.2e-08 6.4e-08)
VIN6 ni6 0 PULSE(0 1.8 3.2e-08 20p 20p 6.4e-08 1.28e-07)
VIN7 ni7 0 PULSE(0 1.8 6.4e-08 20p 20p 1.28e-07 2.56e-07)
VIN8 ni8 0 PULSE(0 1.8 1.28e-07 20p 20p 2.56e-07 5.12e-07)
VIN9 ni9 0 PULSE(0 1.8 2.56e-07 20p 20p 5.12e-07 1.024e-06)
VIN10 nq0 0 PULSE(0 1.8 5.12e-07 20p 20p 1.024e-06 2.048e-06)
VIN11 nq1 0 PULSE(0 1.8 1.024e-06 20p 20p 2.048e-06 4.096e-06)
VIN12 nq2 0 PULSE(0 1.8 2.048e-06 20p 20p 4.096e-06 8.192e-06)
VIN13 nq3 0 PULSE(0 1.8 4.096e-06 20p 20p 8.192e-06 1.6384e-05)
VIN14 nq4 0 PULSE(0 1.8 8.192e-06 20p 20p 1.6384e-05 3.2768e-05)
VIN15 nq5 0 PULSE(0 1.8 1.6384e-05 20p 20p 3.2768e-05 6.5536e-05)
VIN16 nq6 0 PULSE(0 1.8 3.2768e-05 20p 20p 6.5536e-05 0.000131072)
VIN17 nq7 0 PULSE(0 1.8 6.5536e-05 20p 20p 0.000131072 0.000262144)
VIN18 nq8 0 PULSE(0 1.8 0.000131072 20p 20p 0.000262144 0.000524288)
VIN19 nq9 0 PULSE(0 1.8 0.000262144 20p 20p 0.000524288 0.001048576)
VIN20 nq10 0 PULSE(0 1.8 0.000524288 20p 20p 0.001048576 0.002097152)
VIN21 nq11 0 PULSE(0 1.8 0.001048576 20p 20p 0.002097152 0.004194304)
VIN22 nq12 0 PULSE(0 1.8 0.002097152 20p 20p 0.004194304 0.008388608)
VIN23 nq13 0 PULSE(0 1.8 0.004194304 20p 20p 0.008388608 0.016777216)
VIN24 nq14 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN25 nq15 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN26 nq16 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN27 nq17 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN28 nq18 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN29 nq19 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN30 nq20 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
CT1 t1 0 0.1f
CT2 t2 0 0.1f
CT3 t3 0 0.1f
M1 t1 nq0 vdd vdd pch w=2u l=180n
M2 t1 ni0 vdd vdd pch w=2u l=180n
CT4 t4 0 0.1f
M3 t1 nq0 t4 0 nch w=1u l=180n
M4 t4 ni0 0 0 nch w=1u l=180n
M5 t2 nq0 vdd vdd pch w=2u l=180n
M6 t2 t1 vdd vdd pch w=2u l=180n
CT5 t5 0 0.1f
M7 t2 nq0 t5 0 nch w=1u l=180n
M8 t5 t1 0 0 nch w=1u l=180n
M9 t3 ni0 vdd vdd pch w=2u l=180n
M10 t3 t1 vdd vdd pch w=2u l=180n
CT6 t6 0 0.1f
M11 t3 ni0 t6 0 nch w=1u l=180n
M12 t6 t1 0 0 nch w=1u l=180n
M13 nw1 t2 vdd vdd pch w=2u l=180n
M14 nw1 t3 vdd vdd pch w=2u l=180n
CT7 t7 0 0.1f
M15 nw1 t2 t7 0 nch w=1u l=180n
M16 t7 t3 0 0 nch w=1u l=180n
Cnw1 nw1 0 2f
CT8 t8 0 0.1f
M17 t8 ni0 vdd vdd pch w=2u l=180n
M18 t8 nq0 vdd vdd pch w=2u l=180n
CT9 t9 0 0.1f
M19 t8 ni0 t9 0 nch w=1u l=180n
M20 t9 nq0 0 0 nch w=1u l=180n
M21 nw2 t8 vdd vdd pch w=2u l=180n
M22 nw2 t8 0 0 nch w=1u l=180n
Cnw2 nw2 0 2f
CT10 t10 0 0.1f
CT11 t11 0 0.1f
CT12 t12 0 0.1f
M23 t10 nq1 vdd vdd pch w=2u l=180n
M24 t10 nw2 vdd vdd pch w=2u l=180n
CT13 t13 0 0.1f
M25 t10 nq1 t13 0 nch w=1u l=180n
M26 t13 nw2 0 0 nch w=1u l=180n
M27 t11 nq1 vdd vdd pch w=2u l=180n
M28 t11 t10 vdd vdd pch w=2u l=180n
CT14 t14 0 0.1f
M29 t11 nq1 t14 0 nch w=1u l=180n
M30 t14 t10 0 0 nch w=1u l=180n
M31 t12 nw2 vdd vdd pch w=2u l=180n
M32 t12 t10 vdd vdd pch w=2u l=180n
CT15 t15 0 0.1f
M33 t12 nw2 t15 0 nch w=1u l=180n
M34 t15 t10 0 0 nch w=1u l=180n
M35 nw3 t11 vdd vdd pch w=2u l=180n
M36 nw3 t12 vdd vdd pch w=2u l=180n
CT16 t16 0 0.1f
M37 nw3 t11 t16 0 nch w=1u l=180n
M38 t16 t12 0 0 nch w=1u l=180n
Cnw3 nw3 0 2f
CT17 t17 0 0.1f
M39 t17 nw2 vdd vdd pch w=2u l=180n
M40 t17 nq1 vdd vdd pch w=2u l=180n
CT18 t18 0 0.1f
M41 t17 nw2 t18 0 nch w=1u l=180n
M42 t18 nq1 0 0 nch w=1u l=180n
M43 nw4 t17 vdd vdd pch w=2u l=180n
M44 nw4 t17 0 0 nch w=1u l=180n
Cnw4 nw4 0 2f
CT19 t19 0 0.1f
CT20 t20 0 0.1f
CT21 t21 0 0.1f
M45 t19 nq2 vdd vdd pch w=2u l=180n
M46 t19 nw4 vdd vdd pch w=2u l=180n
CT22 t22 0 0.1f
M47 t19 nq2 t22 0 nch w=1u l=180n
M48 t22 nw4 0 0 nch w=1u l=180n
M49 t20 nq2 vdd vdd pch w=2u l=180n
M50 t20 t19 vdd vdd pch w=2u l=180n
CT23 t23 0 0.1f
M51 t20 nq2 t23 0 nch w=1u l=180n
M52 t23 t19 0 0 nch w=1u l=180n
M53 t21 nw4 vdd vdd pch w=2u l=180n
M54 t21 t19 vdd vdd pch w=2u l=180n
CT24 t24 0 0.1f
M55 t21 nw4 t24 0 nch w=1u l=180n
M56 t24 t19 0 0 nch w=1u l=180n
M57 nw5 t20 vdd vdd pch w=2u l=180n
M58 nw5 t21 vdd vdd pch w=2u l=180n
CT25 t25 0 0.1f
M59 nw5 t20 t25 0 nch w=1u l=180n
M60 t25 t21 0 0 nch w=1u l=180n
Cnw5 nw5 0 2f
CT26 t26 0 0.1f
M61 t26 nw4 vdd vdd pch w=2u l=180n
M62 t26 nq2 vdd vdd pch w=2u l=180n
CT27 t27 0 0.1f
M63 t26 nw4 t27 0 nch w=1u l=180n
M64 t27 nq2 0 0 nch w=1u l=180n
M65 nw6 t26 vdd vdd pch w=2u l=180n
M66 nw6 t26 0 0 nch w=1u l=180n
Cnw6 nw6 0 2f
CT28 t28 0 0.1f
CT29 t29 0 0.1f
CT30 t30 0 0.1f
M67 t28 nq3 vdd vdd pch w=2u l=180n
M68 t28 nw6 vdd vdd pch w=2u l=180n
CT31 t31 0 0.1f
M69 t28 nq3 t31 0 nch w=1u l=180n
M70 t31 nw6 0 0 nch w=1u l=180n
M71 t29 nq3 vdd vdd pch w=2u l=180n
M72 t29 t28 vdd vdd pch w=2u l=180n
CT32 t32 0 0.1f
M73 t29 nq3 t32 0 nch w=1u l=180n
M74 t32 t28 0 0 nch w=1u l=180n
M75 t30 nw6 vdd vdd pch w=2u l=180n
M76 t30 t28 vdd vdd pch w=2u l=180n
CT33 t33 0 0.1f
M77 t30 nw6 t33 0 nch w=1u l=180n
M78 t33 t28 0 0 nch w=1u l=180n
M79 nw7 t29 vdd vdd pch w=2u l=180n
M80 nw7 t30 vdd vdd pch w=2u l=180n
CT34 t34 0 0.1f
M81 nw7 t29 t34 0 nch w=1u l=180n
M82 t34 t30 0 0 nch w=1u l=180n
Cnw7 nw7 0 2f
CT35 t35 0 0.1f
M83 t35 nw6 vdd vdd pch w=2u l=180n
M84 t35 nq3 vdd vdd pch w=2u l=180n
CT36 t36 0 0.1f
M85 t35 nw6 t36 0 nch w=1u l=180n
M86 t36 nq3 0 0 nch w=1u l=180n
M87 nw8 t35 vdd vdd pch w=2u l=180n
M88 nw8 t35 0 0 nch w=1u l=180n
Cnw8 nw8 0 2f
CT37 t37 0 0.1f
CT38 t38 0 0.1f
CT39 t39 0 0.1f
M89 t37 nq4 vdd vdd pch w=2u l=180n
M90 t37 nw8 vdd vdd pch w=2u l=180n
CT40 t40 0 0.1f
M91 t37 nq4 t40 0 nch w=1u l=180n
M92 t40 nw8 0 0 nch w=1u l=180n
M93 t38 nq4 vdd vdd pch w=2u l=180n
M94 t38 t37 vdd vdd pch w=2u l=180n
CT41 t41 0 0.1f
M95 t38 nq4 t41 0 nch w=1u l=180n
M96 t41 t37 0 0 nch w=1u l=180n
M97 t39 nw8 vdd vdd pch w=2u l=180n
M98 t39 t37 vdd vdd pch w=2u l=180n
CT42 t42 0 0.1f
M99 t39 nw8 t42 0 nch w=1u l=180n
M100 t42 t37 0 0 nch w=1u l=180n
M101 nw9 t38 vdd vdd pch w=2u l=180n
M102 nw9 t39 vdd vdd pch w=2u l=180n
CT43 t43 0 0.1f
M103 nw9 t38 t43 0 nch w=1u l=180n
M104 t43 t39 0 0 nch w=1u l=180n
Cnw9 nw9 0 2f
CT44 t44 0 0.1f
M105 t44 nw8 vdd vdd pch w=2u l=180n
M106 t44 nq4 vdd vdd pch w=2u l=180n
CT45 t45 0 0.1f
M107 t44 nw8 t45 0 nch w=1u l=180n
M108 t45 nq4 0 0 nch w=1u l=180n
M109 nw10 t44 vdd vdd pch w=2u l=180n
M110 nw10 t44 0 0 nch w=1u l=180n
Cnw10 nw10 0 2f
CT46 t46 0 0.1f
CT47 t47 0 0.1f
CT48 t48 0 0.1f
M111 t46 nq5 vdd vdd pch w=2u l=180n
M112 t46 nw10 vdd vdd pch w=2u l=180n
CT49 t49 0 0.1f
M113 t46 nq5 t49 0 nch w=1u l=180n
M114 t49 nw10 0 0 nch w=1u l=180n
M115 t47 nq5 vdd vdd pch w=2u l=180n
M116 t47 t46 vdd vdd pch w=2u l=180n
CT50 t50 0 0.1f
M117 t47 nq5 t50 0 nch w=1u l=180n
M118 t50 t46 0 0 nch w=1u l=180n
M119 t48 nw10 vdd vdd pch w=2u l=180n
M120 t48 t46 vdd vdd pch w=2u l=180n
CT51 t51 0 0.1f
M121 t48 nw10 t51 0 nch w=1u l=180n
M122 t51 t46 0 0 nch w=1u l=180n
M123 nw11 t47 vdd vdd pch w=2u l=180n
M124 nw11 t48 vdd vdd pch w=2u l=180n
CT52 t52 0 0.1f
M125 nw11 t47 t52 0 nch w=1u l=180n
M126 t52 t48 0 0 nch w=1u l=180n
Cnw11 nw11 0 2f
CT53 t53 0 0.1f
M127 t53 nw10 vdd vdd pch w=2u l=180n
M128 t53 nq5 vdd vdd pch w=2u l=180n
CT54 t54 0 0.1f
M129 t53 nw10 t54 0 nch w=1u l=180n
M130 t54 nq5 0 0 nch w=1u l=180n
M131 nw12 t53 vdd vdd pch w=2u l=180n
M132 nw12 t53 0 0 nch w=1u l=180n
Cnw12 nw12 0 2f
CT55 t55 0 0.1f
CT56 t56 0 0.1f
CT57 t57 0 0.1f
M133 t55 nq6 vdd vdd pch w=2u l=180n
M134 t55 nw12 vdd vdd pch w=2u l=180n
CT58 t58 0 0.1f
M135 t55 nq6 t58 0 nch w=1u l=180n
M136 t58 nw12 0 0 nch w=1u l=180n
M137 t56 nq6 vdd vdd pch w=2u l=180n
M138 t56 t55 vdd vdd pch w=2u l=180n
CT59 t59 0 0.1f
M139 t56 nq6 t59 0 nch w=1u l=180n
M140 t59 t55 0 0 nch w=1u l=180n
M141 t57 nw12 vdd vdd pch w=2u l=180n
M142 t57 t55 vdd vdd pch w=2u l=180n
CT60 t60 0 0.1f
M143 t57 nw12 t60 0 nch w=1u l=180n
M144 t60 t55 0 0 nch w=1u l=180n
M145 nw13 t56 vdd vdd pch w=2u l=180n
M146 nw13 t57 vdd vdd pch w=2u l=180n
CT61 t61 0 0.1f
M147 nw13 t56 t61 0 nch w=1u l=180n
M148 t61 t57 0 0 nch w=1u l=180n
Cnw13 nw13 0 2f
CT62 t62 0 0.1f
M149 t62 nw12 vdd vdd pch w=2u l=180n
M150 t62 nq6 vdd vdd pch w=2u l=180n
CT63 t63 0 0.1f
M151 t62 nw12 t63 0 nch w=1u l=180n
M152 t63 nq6 0 0 nch w=1u l=180n
M153 nw14 t62 vdd vdd pch w=2u l=180n
M154 nw14 t62 0 0 nch w=1u l=180n
Cnw14 nw14 0 2f
CT64 t64 0 0.1f
CT65 t65 0 0.1f
CT66 t66 0 0.1f
M155 t64 nq7 vdd vdd pch w=2u l=180n
M156 t64 nw14 vdd vdd pch w=2u l=180n
CT67 t67 0 0.1f
M157 t64 nq7 t67 0 nch w=1u l=180n
M158 t67 nw14 0 0 nch w=1u l=180n
M159 t65 nq7 vdd vdd pch w=2u l=180n
M160 t65 t64 vdd vdd pch w=2u l=180n
CT68 t68 0 0.1f
M161 t65 nq7 t68 0 nch w=1u l=180n
M162 t68 t64 0 0 nch w=1u l=180n
M163 t66 nw14 vdd vdd pch w=2u l=180n
M164 t66 t64 vdd vdd pch w=2u l=180n
CT69 t69 0 0.1f
M165 t66 nw14 t69 0 nch w=1u l=180n
M166 t69 t64 0 0 nch w=1u l=180n
M167 nw15 t65 vdd vdd pch w=2u l=180n
M168 nw15 t66 vdd vdd pch w=2u l=180n
CT70 t70 0 0.1f
M169 nw15 t65 t70 0 nch w=1u l=180n
M170 t70 t66 0 0 nch w=1u l=180n
Cnw15 nw15 0 2f
CT71 t71 0 0.1f
M171 t71 nw14 vdd vdd pch w=2u l=180n
M172 t71 nq7 vdd vdd pch w=2u l=180n
CT72 t72 0 0.1f
M173 t71 nw14 t72 0 nch w=1u l=180n
M174 t72 nq7 0 0 nch w=1u l=180n
M175 nw16 t71 vdd vdd pch w=2u l=180n
M176 nw16 t71 0 0 nch w=1u l=180n
Cnw16 nw16 0 2f
CT73 t73 0 0.1f
CT74 t74 0 0.1f
CT75 t75 0 0.1f
M177 t73 nq8 vdd vdd pch w=2u l=180n
M178 t73 nw16 vdd vdd pch w=2u l=180n
CT76 t76 0 0.1f
M179 t73 nq8 t76 0 nch w=1u l=180n
M180 t76 nw16 0 0 nch w=1u l=180n
M181 t74 nq8 vdd vdd pch w=2u l=180n
M182 t74 t73 vdd vdd pch w=2u l=180n
CT77 t77 0 0.1f
M183 t74 nq8 t77 0 nch w=1u l=180n
M184 t77 t73 0 0 nch w=1u l=180n
M185 t75 nw16 vdd vdd pch w=2u l=180n
M186 t75 t73 vdd vdd pch w=2u l=180n
CT78 t78 0 0.1f
M187 t75 nw16 t78 0 nch w=1u l=180n
M188 t78 t73 0 0 nch w=1u l=180n
M189 nw17 t74 vdd vdd pch w=2u l=180n
M190 nw17 t75 vdd vdd pch w=2u l=180n
CT79 t79 0 0.1f
M191 nw17 t74 t79 0 nch w=1u l=180n
M192 t79 t75 0 0 nch w=1u l=180n
Cnw17 nw17 0 2f
CT80 t80 0 0.1f
M193 t80 nw16 vdd vdd pch w=2u l=180n
M194 t80 nq8 vdd vdd pch w=2u l=180n
CT81 t81 0 0.1f
M195 t80 nw16 t81 0 nch w=1u l=180n
M196 t81 nq8 0 0 nch w=1u l=180n
M197 nw18 t80 vdd vdd pch w=2u l=180n
M198 nw18 t80 0 0 nch w=1u l=180n
Cnw18 nw18 0 2f
CT82 t82 0 0.1f
CT83 t83 0 0.1f
CT84 t84 0 0.1f
M199 t82 nq9 vdd vdd pch w=2u l=180n
M200 t82 nw18 vdd vdd pch w=2u l=180n
CT85 t85 0 0.1f
M201 t82 nq9 t85 0 nch w=1u l=180n
M202 t85 nw18 0 0 nch w=1u l=180n
M203 t83 nq9 vdd vdd pch w=2u l=180n
M204 t83 t82 vdd vdd pch w=2u l=180n
CT86 t86 0 0.1f
M205 t83 nq9 t86 0 nch w=1u l=180n
M206 t86 t82 0 0 nch w=1u l=180n
M207 t84 nw18 vdd vdd pch w=2u l=180n
M208 t84 t82 vdd vdd pch w=2u l=180n
CT87 t87 0 0.1f
M209 t84 nw18 t87 0 nch w=1u l=180n
M210 t87 t82 0 0 nch w=1u l=180n
M211 nw19 t83 vdd vdd pch w=2u l=180n
M212 nw19 t84 vdd vdd pch w=2u l=180n
CT88 t88 0 0.1f
M213 nw19 t83 t88 0 nch w=1u l=180n
M214 t88 t84 0 0 nch w=1u l=180n
Cnw19 nw19 0 2f
CT89 t89 0 0.1f
M215 t89 nw18 vdd vdd pch w=2u l=180n
M216 t89 nq9 vdd vdd pch w=2u l=180n
CT90 t90 0 0.1f
M217 t89 nw18 t90 0 nch w=1u l=180n
M218 t90 nq9 0 0 nch w=1u l=180n
M219 nw20 t89 vdd vdd pch w=2u l=180n
M220 nw20 t89 0 0 nch w=1u l=180n
Cnw20 nw20 0 2f
CT91 t91 0 0.1f
CT92 t92 0 0.1f
CT93 t93 0 0.1f
M221 t91 nq10 vdd vdd pch w=2u l=180n
M222 t91 nw20 vdd vdd pch w=2u l=180n
CT94 t94 0 0.1f
M223 t91 nq10 t94 0 nch w=1u l=180n
M224 t94 nw20 0 0 nch w=1u l=180n
M225 t92 nq10 vdd vdd pch w=2u l=180n
M226 t92 t91 vdd vdd pch w=2u l=180n
CT95 t95 0 0.1f
M227 t92 nq10 t95 0 nch w=1u l=180n
M228 t95 t91 0 0 nch w=1u l=180n
M229 t93 nw20 vdd vdd pch w=2u l=180n
M230 t93 t91 vdd vdd pch w=2u l=180n
CT96 t96 0 0.1f
M231 t93 nw20 t96 0 nch w=1u l=180n
M232 t96 t91 0 0 nch w=1u l=180n
M233 nw21 t92 vdd vdd pch w=2u l=180n
M234 nw21 t93 vdd vdd pch w=2u l=180n
CT97 t97 0 0.1f
M235 nw21 t92 t97 0 nch w=1u l=180n
M236 t97 t93 0 0 nch w=1u l=180n
Cnw21 nw21 0 2f
CT98 t98 0 0.1f
M237 t98 nw20 vdd vdd pch w=2u l=180n
M238 t98 nq10 vdd vdd pch w=2u l=180n
CT99 t99 0 0.1f
M239 t98 nw20 t99 0 nch w=1u l=180n
M240 t99 nq10 0 0 nch w=1u l=180n
M241 nw22 t98 vdd vdd pch w=2u l=180n
M242 nw22 t98 0 0 nch w=1u l=180n
Cnw22 nw22 0 2f
CT100 t100 0 0.1f
CT101 t101 0 0.1f
CT102 t102 0 0.1f
M243 t100 nq11 vdd vdd pch w=2u l=180n
M244 t100 nw22 vdd vdd pch w=2u l=180n
CT103 t103 0 0.1f
M245 t100 nq11 t103 0 nch w=1u l=180n
M246 t103 nw22 0 0 nch w=1u l=180n
M247 t101 nq11 vdd vdd pch w=2u l=180n
M248 t101 t100 vdd vdd pch w=2u l=180n
CT104 t104 0 0.1f
M249 t101 nq11 t104 0 nch w=1u l=180n
M250 t104 t100 0 0 nch w=1u l=180n
M251 t102 nw22 vdd vdd pch w=2u l=180n
M252 t102 t100 vdd vdd pch w=2u l=180n
CT105 t105 0 0.1f
M253 t102 nw22 t105 0 nch w=1u l=180n
M254 t105 t100 0 0 nch w=1u l=180n
M255 nw23 t101 vdd vdd pch w=2u l=180n
M256 nw23 t102 vdd vdd pch w=2u l=180n
CT106 t106 0 0.1f
M257 nw23 t101 t106 0 nch w=1u l=180n
M258 t106 t102 0 0 nch w=1u l=180n
Cnw23 nw23 0 2f
CT107 t107 0 0.1f
M259 t107 nw22 vdd vdd pch w=2u l=180n
M260 t107 nq11 vdd vdd pch w=2u l=180n
CT108 t108 0 0.1f
M261 t107 nw22 t108 0 nch w=1u l=180n
M262 t108 nq11 0 0 nch w=1u l=180n
M263 nw24 t107 vdd vdd pch w=2u l=180n
M264 nw24 t107 0 0 nch w=1u l=180n
Cnw24 nw24 0 2f
CT109 t109 0 0.1f
CT110 t110 0 0.1f
CT111 t111 0 0.1f
M265 t109 nq12 vdd vdd pch w=2u l=180n
M266 t109 nw24 vdd vdd pch w=2u l=180n
CT112 t112 0 0.1f
M267 t109 nq12 t112 0 nch w=1u l=180n
M268 t112 nw24 0 0 nch w=1u l=180n
M269 t110 nq12 vdd vdd pch w=2u l=180n
M270 t110 t109 vdd vdd pch w=2u l=180n
CT113 t113 0 0.1f
M271 t110 nq12 t113 0 nch w=1u l=180n
M272 t113 t109 0 0 nch w=1u l=180n
M273 t111 nw24 vdd vdd pch w=2u l=180n
M274 t111 t109 vdd vdd pch w=2u l=180n
CT114 t114 0 0.1f
M275 t111 nw24 t114 0 nch w=1u l=180n
M276 t114 t109 0 0 nch w=1u l=180n
M277 nw25 t110 vdd vdd pch w=2u l=180n
M278 nw25 t111 vdd vdd pch w=2u l=180n
CT115 t115 0 0.1f
M279 nw25 t110 t115 0 nch w=1u l=180n
M280 t115 t111 0 0 nch w=1u l=180n
Cnw25 nw25 0 2f
CT116 t116 0 0.1f
M281 t116 nw24 vdd vdd pch w=2u l=180n
M282 t116 nq12 vdd vdd pch w=2u l=180n
CT117 t117 0 0.1f
M283 t116 nw24 t117 0 nch w=1u l=180n
M284 t117 nq12 0 0 nch w=1u l=180n
M285 nw26 t116 vdd vdd pch w=2u l=180n
M286 nw26 t116 0 0 nch w=1u l=180n
Cnw26 nw26 0 2f
CT118 t118 0 0.1f
CT119 t119 0 0.1f
CT120 t120 0 0.1f
M287 t118 nq13 vdd vdd pch w=2u l=180n
M288 t118 nw26 vdd vdd pch w=2u l=180n
CT121 t121 0 0.1f
M289 t118 nq13 t121 0 nch w=1u l=180n
M290 t121 nw26 0 0 nch w=1u l=180n
M291 t119 nq13 vdd vdd pch w=2u l=180n
M292 t119 t118 vdd vdd pch w=2u l=180n
CT122 t122 0 0.1f
M293 t119 nq13 t122 0 nch w=1u l=180n
M294 t122 t118 0 0 nch w=1u l=180n
M295 t120 nw26 vdd vdd pch w=2u l=180n
M296 t120 t118 vdd vdd pch w=2u l=180n
CT123 t123 0 0.1f
M297 t120 nw26 t123 0 nch w=1u l=180n
M298 t123 t118 0 0 nch w=1u l=180n
M299 nw27 t119 vdd vdd pch w=2u l=180n
M300 nw27 t120 vdd vdd pch w=2u l=180n
CT124 t124 0 0.1f
M301 nw27 t119 t124 0 nch w=1u l=180n
M302 t124 t120 0 0 nch w=1u l=180n
Cnw27 nw27 0 2f
CT125 t125 0 0.1f
M303 t125 nw26 vdd vdd pch w=2u l=180n
M304 t125 nq13 vdd vdd pch w=2u l=180n
CT126 t126 0 0.1f
M305 t125 nw26 t126 0 nch w=1u l=180n
M306 t126 nq13 0 0 nch w=1u l=180n
M307 nw28 t125 vdd vdd pch w=2u l=180n
M308 nw28 t125 0 0 nch w=1u l=180n
Cnw28 nw28 0 2f
CT127 t127 0 0.1f
CT128 t128 0 0.1f
CT129 t129 0 0.1f
M309 t127 nq14 vdd vdd pch w=2u l=180n
M310 t127 nw28 vdd vdd pch w=2u l=180n
CT130 t130 0 0.1f
M311 t127 nq14 t130 0 nch w=1u l=180n
M312 t130 nw28 0 0 nch w=1u l=180n
M313 t128 nq14 vdd vdd pch w=2u l=180n
M314 t128 t127 vdd vdd pch w=2u l=180n
CT131 t131 0 0.1f
M315 t128 nq14 t131 0 nch w=1u l=180n
M316 t131 t127 0 0 nch w=1u l=180n
M317 t129 nw28 vdd vdd pch w=2u l=180n
M318 t129 t127 vdd vdd pch w=2u l=180n
CT132 t132 0 0.1f
M319 t129 nw28 t132 0 nch w=1u l=180n
M320 t132 t127 0 0 nch w=1u l=180n
M321 nw29 t128 vdd vdd pch w=2u l=180n
M322 nw29 t129 vdd vdd pch w=2u l=180n
CT133 t133 0 0.1f
M323 nw29 t128 t133 0 nch w=1u l=180n
M324 t133 t129 0 0 nch w=1u l=180n
Cnw29 nw29 0 2f
CT134 t134 0 0.1f
M325 t134 nw28 vdd vdd pch w=2u l=180n
M326 t134 nq14 vdd vdd pch w=2u l=180n
CT135 t135 0 0.1f
M327 t134 nw28 t135 0 nch w=1u l=180n
M328 t135 nq14 0 0 nch w=1u l=180n
M329 nw30 t134 vdd vdd pch w=2u l=180n
M330 nw30 t134 0 0 nch w=1u l=180n
Cnw30 nw30 0 2f
CT136 t136 0 0.1f
CT137 t137 0 0.1f
CT138 t138 0 0.1f
M331 t136 nq15 vdd vdd pch w=2u l=180n
M332 t136 nw30 vdd vdd pch w=2u l=180n
CT139 t139 0 0.1f
M333 t136 nq15 t139 0 nch w=1u l=180n
M334 t139 nw30 0 0 nch w=1u l=180n
M335 t137 nq15 vdd vdd pch w=2u l=180n
M336 t137 t136 vdd vdd pch w=2u l=180n
CT140 t140 0 0.1f
M337 t137 nq15 t140 0 nch w=1u l=180n
M338 t140 t136 0 0 nch w=1u l=180n
M339 t138 nw30 vdd vdd pch w=2u l=180n
M340 t138 t136 vdd vdd pch w=2u l=180n
CT141 t141 0 0.1f
M341 t138 nw30 t141 0 nch w=1u l=180n
M342 t141 t136 0 0 nch w=1u l=180n
M343 nw31 t137 vdd vdd pch w=2u l=180n
M344 nw31 t138 vdd vdd pch w=2u l=180n
CT142 t142 0 0.1f
M345 nw31 t137 t142 0 nch w=1u l=180n
M346 t142 t138 0 0 nch w=1u l=180n
Cnw31 nw31 0 2f
CT143 t143 0 0.1f
M347 t143 nw30 vdd vdd pch w=2u l=180n
M348 t143 nq15 vdd vdd pch w=2u l=180n
CT144 t144 0 0.1f
M349 t143 nw30 t144 0 nch w=1u l=180n
M350 t144 nq15 0 0 nch w=1u l=180n
M351 nw32 t143 vdd vdd pch w=2u l=180n
M352 nw32 t143 0 0 nch w=1u l=180n
Cnw32 nw32 0 2f
CT145 t145 0 0.1f
CT146 t146 0 0.1f
CT147 t147 0 0.1f
M353 t145 nq16 vdd vdd pch w=2u l=180n
M354 t145 nw32 vdd vdd pch w=2u l=180n
CT148 t148 0 0.1f
M355 t145 nq16 t148 0 nch w=1u l=180n
M356 t148 nw32 0 0 nch w=1u l=180n
M357 t146 nq16 vdd vdd pch w=2u l=180n
M358 t146 t145 vdd vdd pch w=2u l=180n
CT149 t149 0 0.1f
M359 t146 nq16 t149 0 nch w=1u l=180n
M360 t149 t145 0 0 nch w=1u l=180n
M361 t147 nw32 vdd vdd pch w=2u l=180n
M362 t147 t145 vdd vdd pch w=2u l=180n
CT150 t150 0 0.1f
M363 t147 nw32 t150 0 nch w=1u l=180n
M364 t150 t145 0 0 nch w=1u l=180n
M365 nw33 t146 vdd vdd pch w=2u l=180n
M366 nw33 t147 vdd vdd pch w=2u l=180n
CT151 t151 0 0.1f
M367 nw33 t146 t151 0 nch w=1u l=180n
M368 t151 t147 0 0 nch w=1u l=180n
Cnw33 nw33 0 2f
CT152 t152 0 0.1f
M369 t152 nw32 vdd vdd pch w=2u l=180n
M370 t152 nq16 vdd vdd pch w=2u l=180n
CT153 t153 0 0.1f
M371 t152 nw32 t153 0 nch w=1u l=180n
M372 t153 nq16 0 0 nch w=1u l=180n
M373 nw34 t152 vdd vdd pch w=2u l=180n
M374 nw34 t152 0 0 nch w=1u l=180n
Cnw34 nw34 0 2f
CT154 t154 0 0.1f
CT155 t155 0 0.1f
CT156 t156 0 0.1f
M375 t154 nq17 vdd vdd pch w=2u l=180n
M376 t154 nw34 vdd vdd pch w=2u l=180n
CT157 t157 0 0.1f
M377 t154 nq17 t157 0 nch w=1u l=180n
M378 t157 nw34 0 0 nch w=1u l=180n
M379 t155 nq17 vdd vdd pch w=2u l=180n
M380 t155 t154 vdd vdd pch w=2u l=180n
CT158 t158 0 0.1f
M381 t155 nq17 t158 0 nch w=1u l=180n
M382 t158 t154 0 0 nch w=1u l=180n
M383 t156 nw34 vdd vdd pch w=2u l=180n
M384 t156 t154 vdd vdd pch w=2u l=180n
CT159 t159 0 0.1f
M385 t156 nw34 t159 0 nch w=1u l=180n
M386 t159 t154 0 0 nch w=1u l=180n
M387 nw35 t155 vdd vdd pch w=2u l=180n
M388 nw35 t156 vdd vdd pch w=2u l=180n
CT160 t160 0 0.1f
M389 nw35 t155 t160 0 nch w=1u l=180n
M390 t160 t156 0 0 nch w=1u l=180n
Cnw35 nw35 0 2f
CT161 t161 0 0.1f
M391 t161 nw34 vdd vdd pch w=2u l=180n
M392 t161 nq17 vdd vdd pch w=2u l=180n
CT162 t162 0 0.1f
M393 t161 nw34 t162 0 nch w=1u l=180n
M394 t162 nq17 0 0 nch w=1u l=180n
M395 nw36 t161 vdd vdd pch w=2u l=180n
M396 nw36 t161 0 0 nch w=1u l=180n
Cnw36 nw36 0 2f
CT163 t163 0 0.1f
CT164 t164 0 0.1f
CT165 t165 0 0.1f
M397 t163 nq18 vdd vdd pch w=2u l=180n
M398 t163 nw36 vdd vdd pch w=2u l=180n
CT166 t166 0 0.1f
M399 t163 nq18 t166 0 nch w=1u l=180n
M400 t166 nw36 0 0 nch w=1u l=180n
M401 t164 nq18 vdd vdd pch w=2u l=180n
M402 t164 t163 vdd vdd pch w=2u l=180n
CT167 t167 0 0.1f
M403 t164 nq18 t167 0 nch w=1u l=180n
M404 t167 t163 0 0 nch w=1u l=180n
M405 t165 nw36 vdd vdd pch w=2u l=180n
M406 t165 t163 vdd vdd pch w=2u l=180n
CT168 t168 0 0.1f
M407 t165 nw36 t168 0 nch w=1u l=180n
M408 t168 t163 0 0 nch w=1u l=180n
M409 nw37 t164 vdd vdd pch w=2u l=180n
M410 nw37 t165 vdd vdd pch w=2u l=180n
CT169 t169 0 0.1f
M411 nw37 t164 t169 0 nch w=1u l=180n
M412 t169 t165 0 0 nch w=1u l=180n
Cnw37 nw37 0 2f
CT170 t170 0 0.1f
M413 t170 nw36 vdd vdd pch w=2u l=180n
M414 t170 nq18 vdd vdd pch w=2u l=180n
CT171 t171 0 0.1f
M415 t170 nw36 t171 0 nch w=1u l=180n
M416 t171 nq18 0 0 nch w=1u l=180n
M417 nw38 t170 vdd vdd pch w=2u l=180n
M418 nw38 t170 0 0 nch w=1u l=180n
Cnw38 nw38 0 2f
CT172 t172 0 0.1f
CT173 t173 0 0.1f
CT174 t174 0 0.1f
M419 t172 nq19 vdd vdd pch w=2u l=180n
M420 t172 nw38 vdd vdd pch w=2u l=180n
CT175 t175 0 0.1f
M421 t172 nq19 t175 0 nch w=1u l=180n
M422 t175 nw38 0 0 nch w=1u l=180n
M423 t173 nq19 vdd vdd pch w=2u l=180n
M424 t173 t172 vdd vdd pch w=2u l=180n
CT176 t176 0 0.1f
M425 t173 nq19 t176 0 nch w=1u l=180n
M426 t176 t172 0 0 nch w=1u l=180n
M427 t174 nw38 vdd vdd pch w=2u l=180n
M428 t174 t172 vdd vdd pch w=2u l=180n
CT177 t177 0 0.1f
M429 t174 nw38 t177 0 nch w=1u l=180n
M430 t177 t172 0 0 nch w=1u l=180n
M431 nw39 t173 vdd vdd pch w=2u l=180n
M432 nw39 t174 vdd vdd pch w=2u l=180n
CT178 t178 0 0.1f
M433 nw39 t173 t178 0 nch w=1u l=180n
M434 t178 t174 0 0 nch w=1u l=180n
Cnw39 nw39 0 2f
CT179 t179 0 0.1f
M435 t179 nw38 vdd vdd pch w=2u l=180n
M436 t179 nq19 vdd vdd pch w=2u l=180n
CT180 t180 0 0.1f
M437 t179 nw38 t180 0 nch w=1u l=180n
M438 t180 nq19 0 0 nch w=1u l=180n
M439 nw40 t179 vdd vdd pch w=2u l=180n
M440 nw40 t179 0 0 nch w=1u l=180n
Cnw40 nw40 0 2f
CT181 t181 0 0.1f
CT182 t182 0 0.1f
CT183 t183 0 0.1f
M441 t181 nq20 vdd vdd pch w=2u l=180n
M442 t181 nw40 vdd vdd pch w=2u l=180n
CT184 t184 0 0.1f
M443 t181 nq20 t184 0 nch w=1u l=180n
M444 t184 nw40 0 0 nch w=1u l=180n
M445 t182 nq20 vdd vdd pch w=2u l=180n
M446 t182 t181 vdd vdd pch w=2u l=180n
CT185 t185 0 0.1f
M447 t182 nq20 t185 0 nch w=1u l=180n
M448 t185 t181 0 0 nch w=1u l=180n
M449 t183 nw40 vdd vdd pch w=2u l=180n
M450 t183 t181 vdd vdd pch w=2u l=180n
CT186 t186 0 0.1f
M451 t183 nw40 t186 0 nch w=1u l=180n
M452 t186 t181 0 0 nch w=1u l=180n
M453 nw41 t182 vdd vdd pch w=2u l=180n
M454 nw41 t183 vdd vdd pch w=2u l=180n
CT187 t187 0 0.1f
M455 nw41 t182 t187 0 nch w=1u l=180n
M456 t187 t183 0 0 nch w=1u l=180n
Cnw41 nw41 0 2f
CT188 t188 0 0.1f
M457 t188 nw40 vdd vdd pch w=2u l=180n
M458 t188 nq20 vdd vdd pch w=2u l=180n
CT189 t189 0 0.1f
M459 t188 nw40 t189 0 nch w=1u l=180n
M460 t189 nq20 0 0 nch w=1u l=180n
M461 nw42 t188 vdd vdd pch w=2u l=180n
M462 nw42 t188 0 0 nch w=1u l=180n
Cnw42 nw42 0 2f
M463 nw43 nq1 vdd vdd pch w=2u l=180n
M464 nw43 nq3 vdd vdd pch w=2u l=180n
CT190 t190 0 0.1f
M465 nw43 nq1 t190 0 nch w=1u l=180n
M466 t190 nq3 0 0 nch w=1u l=180n
Cnw43 nw43 0 2f
M467 nw44 nq8 0 0 nch w=1u l=180n
M468 nw44 nq14 0 0 nch w=1u l=180n
CT191 t191 0 0.1f
M469 t191 nq8 vdd vdd pch w=2u l=180n
M470 nw44 nq14 t191 vdd pch w=2u l=180n
Cnw44 nw44 0 2f
CT192 t192 0 0.1f
M471 t192 nq15 vdd vdd pch w=2u l=180n
M472 t192 ni4 vdd vdd pch w=2u l=180n
CT193 t193 0 0.1f
M473 t192 nq15 t193 0 nch w=1u l=180n
M474 t193 ni4 0 0 nch w=1u l=180n
M475 nw45 t192 vdd vdd pch w=2u l=180n
M476 nw45 t192 0 0 nch w=1u l=180n
Cnw45 nw45 0 2f
CT194 t194 0 0.1f
M477 t194 ni1 0 0 nch w=1u l=180n
M478 t194 nq2 0 0 nch w=1u l=180n
CT195 t195 0 0.1f
M479 t195 ni1 vdd vdd pch w=2u l=180n
M480 t194 nq2 t195 vdd pch w=2u l=180n
M481 nw46 t194 vdd vdd pch w=2u l=180n
M482 nw46 t194 0 0 nch w=1u l=180n
Cnw46 nw46 0 2f
CT196 t196 0 0.1f
CT197 t197 0 0.1f
CT198 t198 0 0.1f
M483 t196 ni8 vdd vdd pch w=2u l=180n
M484 t196 nq12 vdd vdd pch w=2u l=180n
CT199 t199 0 0.1f
M485 t196 ni8 t199 0 nch w=1u l=180n
M486 t199 nq12 0 0 nch w=1u l=180n
M487 t197 ni8 vdd vdd pch w=2u l=180n
M488 t197 t196 vdd vdd pch w=2u l=180n
CT200 t200 0 0.1f
M489 t197 ni8 t200 0 nch w=1u l=180n
M490 t200 t196 0 0 nch w=1u l=180n
M491 t198 nq12 vdd vdd pch w=2u l=180n
M492 t198 t196 vdd vdd pch w=2u l=180n
CT201 t201 0 0.1f
M493 t198 nq12 t201 0 nch w=1u l=180n
M494 t201 t196 0 0 nch w=1u l=180n
M495 nw47 t197 vdd vdd pch w=2u l=180n
M496 nw47 t198 vdd vdd pch w=2u l=180n
CT202 t202 0 0.1f
M497 nw47 t197 t202 0 nch w=1u l=180n
M498 t202 t198 0 0 nch w=1u l=180n
Cnw47 nw47 0 2f
M499 nw48 nq0 vdd vdd pch w=2u l=180n
M500 nw48 ni1 vdd vdd pch w=2u l=180n
CT203 t203 0 0.1f
M501 nw48 nq0 t203 0 nch w=1u l=180n
M502 t203 ni1 0 0 nch w=1u l=180n
Cnw48 nw48 0 2f
M503 nw49 nq6 0 0 nch w=1u l=180n
M504 nw49 nw44 0 0 nch w=1u l=180n
CT204 t204 0 0.1f
M505 t204 nq6 vdd vdd pch w=2u l=180n
M506 nw49 nw44 t204 vdd pch w=2u l=180n
Cnw49 nw49 0 2f
CT205 t205 0 0.1f
M507 t205 nq12 vdd vdd pch w=2u l=180n
M508 t205 nq4 vdd vdd pch w=2u l=180n
CT206 t206 0 0.1f
M509 t205 nq12 t206 0 nch w=1u l=180n
M510 t206 nq4 0 0 nch w=1u l=180n
M511 nw50 t205 vdd vdd pch w=2u l=180n
M512 nw50 t205 0 0 nch w=1u l=180n
Cnw50 nw50 0 2f
CT207 t207 0 0.1f
M513 t207 nq18 0 0 nch w=1u l=180n
M514 t207 nq13 0 0 nch w=1u l=180n
CT208 t208 0 0.1f
M515 t208 nq18 vdd vdd pch w=2u l=180n
M516 t207 nq13 t208 vdd pch w=2u l=180n
M517 nw51 t207 vdd vdd pch w=2u l=180n
M518 nw51 t207 0 0 nch w=1u l=180n
Cnw51 nw51 0 2f
CT209 t209 0 0.1f
CT210 t210 0 0.1f
CT211 t211 0 0.1f
M519 t209 ni3 vdd vdd pch w=2u l=180n
M520 t209 ni1 vdd vdd pch w=2u l=180n
CT212 t212 0 0.1f
M521 t209 ni3 t212 0 nch w=1u l=180n
M522 t212 ni1 0 0 nch w=1u l=180n
M523 t210 ni3 vdd vdd pch w=2u l=180n
M524 t210 t209 vdd vdd pch w=2u l=180n
CT213 t213 0 0.1f
M525 t210 ni3 t213 0 nch w=1u l=180n
M526 t213 t209 0 0 nch w=1u l=180n
M527 t211 ni1 vdd vdd pch w=2u l=180n
M528 t211 t209 vdd vdd pch w=2u l=180n
CT214 t214 0 0.1f
M529 t211 ni1 t214 0 nch w=1u l=180n
M530 t214 t209 0 0 nch w=1u l=180n
M531 nw52 t210 vdd vdd pch w=2u l=180n
M532 nw52 t211 vdd vdd pch w=2u l=180n
CT215 t215 0 0.1f
M533 nw52 t210 t215 0 nch w=1u l=180n
M534 t215 t211 0 0 nch w=1u l=180n
Cnw52 nw52 0 2f
M535 nw53 ni9 vdd vdd pch w=2u l=180n
M536 nw53 nw43 vdd vdd pch w=2u l=180n
CT216 t216 0 0.1f
M537 nw53 ni9 t216 0 nch w=1u l=180n
M538 t216 nw43 0 0 nch w=1u l=180n
Cnw53 nw53 0 2f
M539 nw54 nw48 0 0 nch w=1u l=180n
M540 nw54 nw52 0 0 nch w=1u l=180n
CT217 t217 0 0.1f
M541 t217 nw48 vdd vdd pch w=2u l=180n
M542 nw54 nw52 t217 vdd pch w=2u l=180n
Cnw54 nw54 0 2f
CT218 t218 0 0.1f
M543 t218 nw54 vdd vdd pch w=2u l=180n
M544 t218 nq6 vdd vdd pch w=2u l=180n
CT219 t219 0 0.1f
M545 t218 nw54 t219 0 nch w=1u l=180n
M546 t219 nq6 0 0 nch w=1u l=180n
M547 nw55 t218 vdd vdd pch w=2u l=180n
M548 nw55 t218 0 0 nch w=1u l=180n
Cnw55 nw55 0 2f
CT220 t220 0 0.1f
M549 t220 nq4 0 0 nch w=1u l=180n
M550 t220 nq14 0 0 nch w=1u l=180n
CT221 t221 0 0.1f
M551 t221 nq4 vdd vdd pch w=2u l=180n
M552 t220 nq14 t221 vdd pch w=2u l=180n
M553 nw56 t220 vdd vdd pch w=2u l=180n
M554 nw56 t220 0 0 nch w=1u l=180n
Cnw56 nw56 0 2f
CT222 t222 0 0.1f
CT223 t223 0 0.1f
CT224 t224 0 0.1f
M555 t222 nq9 vdd vdd pch w=2u l=180n
M556 t222 ni1 vdd vdd pch w=2u l=180n
CT225 t225 0 0.1f
M557 t222 nq9 t225 0 nch w=1u l=180n
M558 t225 ni1 0 0 nch w=1u l=180n
M559 t223 nq9 vdd vdd pch w=2u l=180n
M560 t223 t222 vdd vdd pch w=2u l=180n
CT226 t226 0 0.1f
M561 t223 nq9 t226 0 nch w=1u l=180n
M562 t226 t222 0 0 nch w=1u l=180n
M563 t224 ni1 vdd vdd pch w=2u l=180n
M564 t224 t222 vdd vdd pch w=2u l=180n
CT227 t227 0 0.1f
M565 t224 ni1 t227 0 nch w=1u l=180n
M566 t227 t222 0 0 nch w=1u l=180n
M567 nw57 t223 vdd vdd pch w=2u l=180n
M568 nw57 t224 vdd vdd pch w=2u l=180n
CT228 t228 0 0.1f
M569 nw57 t223 t228 0 nch w=1u l=180n
M570 t228 t224 0 0 nch w=1u l=180n
Cnw57 nw57 0 2f
M571 nw58 nq14 vdd vdd pch w=2u l=180n
M572 nw58 ni9 vdd vdd pch w=2u l=180n
CT229 t229 0 0.1f
M573 nw58 nq14 t229 0 nch w=1u l=180n
M574 t229 ni9 0 0 nch w=1u l=180n
Cnw58 nw58 0 2f
M575 nw59 nq19 0 0 nch w=1u l=180n
M576 nw59 nw50 0 0 nch w=1u l=180n
CT230 t230 0 0.1f
M577 t230 nq19 vdd vdd pch w=2u l=180n
M578 nw59 nw50 t230 vdd pch w=2u l=180n
Cnw59 nw59 0 2f
CT231 t231 0 0.1f
M579 t231 ni3 vdd vdd pch w=2u l=180n
M580 t231 nw58 vdd vdd pch w=2u l=180n
CT232 t232 0 0.1f
M581 t231 ni3 t232 0 nch w=1u l=180n
M582 t232 nw58 0 0 nch w=1u l=180n
M583 nw60 t231 vdd vdd pch w=2u l=180n
M584 nw60 t231 0 0 nch w=1u l=180n
Cnw60 nw60 0 2f
CT233 t233 0 0.1f
M585 t233 ni8 0 0 nch w=1u l=180n
M586 t233 nq5 0 0 nch w=1u l=180n
CT234 t234 0 0.1f
M587 t234 ni8 vdd vdd pch w=2u l=180n
M588 t233 nq5 t234 vdd pch w=2u l=180n
M589 nw61 t233 vdd vdd pch w=2u l=180n
M590 nw61 t233 0 0 nch w=1u l=180n
Cnw61 nw61 0 2f
CT235 t235 0 0.1f
CT236 t236 0 0.1f
CT237 t237 0 0.1f
M591 t235 nw46 vdd vdd pch w=2u l=180n
M592 t235 nq12 vdd vdd pch w=2u l=180n
CT238 t238 0 0.1f
M593 t235 nw46 t238 0 nch w=1u l=180n
M594 t238 nq12 0 0 nch w=1u l=180n
M595 t236 nw46 vdd vdd pch w=2u l=180n
M596 t236 t235 vdd vdd pch w=2u l=180n
CT239 t239 0 0.1f
M597 t236 nw46 t239 0 nch w=1u l=180n
M598 t239 t235 0 0 nch w=1u l=180n
M599 t237 nq12 vdd vdd pch w=2u l=180n
M600 t237 t235 vdd vdd pch w=2u l=180n
CT240 t240 0 0.1f
M601 t237 nq12 t240 0 nch w=1u l=180n
M602 t240 t235 0 0 nch w=1u l=180n
M603 nw62 t236 vdd vdd pch w=2u l=180n
M604 nw62 t237 vdd vdd pch w=2u l=180n
CT241 t241 0 0.1f
M605 nw62 t236 t241 0 nch w=1u l=180n
M606 t241 t237 0 0 nch w=1u l=180n
Cnw62 nw62 0 2f
M607 nw63 nw51 vdd vdd pch w=2u l=180n
M608 nw63 nq19 vdd vdd pch w=2u l=180n
CT242 t242 0 0.1f
M609 nw63 nw51 t242 0 nch w=1u l=180n
M610 t242 nq19 0 0 nch w=1u l=180n
Cnw63 nw63 0 2f
M611 nw64 nw56 0 0 nch w=1u l=180n
M612 nw64 ni5 0 0 nch w=1u l=180n
CT243 t243 0 0.1f
M613 t243 nw56 vdd vdd pch w=2u l=180n
M614 nw64 ni5 t243 vdd pch w=2u l=180n
Cnw64 nw64 0 2f
CT244 t244 0 0.1f
M615 t244 nw61 vdd vdd pch w=2u l=180n
M616 t244 nw45 vdd vdd pch w=2u l=180n
CT245 t245 0 0.1f
M617 t244 nw61 t245 0 nch w=1u l=180n
M618 t245 nw45 0 0 nch w=1u l=180n
M619 nw65 t244 vdd vdd pch w=2u l=180n
M620 nw65 t244 0 0 nch w=1u l=180n
Cnw65 nw65 0 2f
CT246 t246 0 0.1f
M621 t246 nq0 0 0 nch w=1u l=180n
M622 t246 nw52 0 0 nch w=1u l=180n
CT247 t247 0 0.1f
M623 t247 nq0 vdd vdd pch w=2u l=180n
M624 t246 nw52 t247 vdd pch w=2u l=180n
M625 nw66 t246 vdd vdd pch w=2u l=180n
M626 nw66 t246 0 0 nch w=1u l=180n
Cnw66 nw66 0 2f
CT248 t248 0 0.1f
CT249 t249 0 0.1f
CT250 t250 0 0.1f
M627 t248 nq4 vdd vdd pch w=2u l=180n
M628 t248 nw59 vdd vdd pch w=2u l=180n
CT251 t251 0 0.1f
M629 t248 nq4 t251 0 nch w=1u l=180n
M630 t251 nw59 0 0 nch w=1u l=180n
M631 t249 nq4 vdd vdd pch w=2u l=180n
M632 t249 t248 vdd vdd pch w=2u l=180n
CT252 t252 0 0.1f
M633 t249 nq4 t252 0 nch w=1u l=180n
M634 t252 t248 0 0 nch w=1u l=180n
M635 t250 nw59 vdd vdd pch w=2u l=180n
M636 t250 t248 vdd vdd pch w=2u l=180n
CT253 t253 0 0.1f
M637 t250 nw59 t253 0 nch w=1u l=180n
M638 t253 t248 0 0 nch w=1u l=180n
M639 nw67 t249 vdd vdd pch w=2u l=180n
M640 nw67 t250 vdd vdd pch w=2u l=180n
CT254 t254 0 0.1f
M641 nw67 t249 t254 0 nch w=1u l=180n
M642 t254 t250 0 0 nch w=1u l=180n
Cnw67 nw67 0 2f
M643 nw68 nq8 vdd vdd pch w=2u l=180n
M644 nw68 nw66 vdd vdd pch w=2u l=180n
CT255 t255 0 0.1f
M645 nw68 nq8 t255 0 nch w=1u l=180n
M646 t255 nw66 0 0 nch w=1u l=180n
Cnw68 nw68 0 2f
M647 nw69 nq12 0 0 nch w=1u l=180n
M648 nw69 nq4 0 0 nch w=1u l=180n
CT256 t256 0 0.1f
M649 t256 nq12 vdd vdd pch w=2u l=180n
M650 nw69 nq4 t256 vdd pch w=2u l=180n
Cnw69 nw69 0 2f
CT257 t257 0 0.1f
M651 t257 nq16 vdd vdd pch w=2u l=180n
M652 t257 nq10 vdd vdd pch w=2u l=180n
CT258 t258 0 0.1f
M653 t257 nq16 t258 0 nch w=1u l=180n
M654 t258 nq10 0 0 nch w=1u l=180n
M655 nw70 t257 vdd vdd pch w=2u l=180n
M656 nw70 t257 0 0 nch w=1u l=180n
Cnw70 nw70 0 2f
CT259 t259 0 0.1f
M657 t259 nq20 0 0 nch w=1u l=180n
M658 t259 nq16 0 0 nch w=1u l=180n
CT260 t260 0 0.1f
M659 t260 nq20 vdd vdd pch w=2u l=180n
M660 t259 nq16 t260 vdd pch w=2u l=180n
M661 nw71 t259 vdd vdd pch w=2u l=180n
M662 nw71 t259 0 0 nch w=1u l=180n
Cnw71 nw71 0 2f
CT261 t261 0 0.1f
CT262 t262 0 0.1f
CT263 t263 0 0.1f
M663 t261 ni3 vdd vdd pch w=2u l=180n
M664 t261 ni1 vdd vdd pch w=2u l=180n
CT264 t264 0 0.1f
M665 t261 ni3 t264 0 nch w=1u l=180n
M666 t264 ni1 0 0 nch w=1u l=180n
M667 t262 ni3 vdd vdd pch w=2u l=180n
M668 t262 t261 vdd vdd pch w=2u l=180n
CT265 t265 0 0.1f
M669 t262 ni3 t265 0 nch w=1u l=180n
M670 t265 t261 0 0 nch w=1u l=180n
M671 t263 ni1 vdd vdd pch w=2u l=180n
M672 t263 t261 vdd vdd pch w=2u l=180n
CT266 t266 0 0.1f
M673 t263 ni1 t266 0 nch w=1u l=180n
M674 t266 t261 0 0 nch w=1u l=180n
M675 nw72 t262 vdd vdd pch w=2u l=180n
M676 nw72 t263 vdd vdd pch w=2u l=180n
CT267 t267 0 0.1f
M677 nw72 t262 t267 0 nch w=1u l=180n
M678 t267 t263 0 0 nch w=1u l=180n
Cnw72 nw72 0 2f
M679 nw73 ni7 vdd vdd pch w=2u l=180n
M680 nw73 ni8 vdd vdd pch w=2u l=180n
CT268 t268 0 0.1f
M681 nw73 ni7 t268 0 nch w=1u l=180n
M682 t268 ni8 0 0 nch w=1u l=180n
Cnw73 nw73 0 2f
M683 nw74 nw44 0 0 nch w=1u l=180n
M684 nw74 nw46 0 0 nch w=1u l=180n
CT269 t269 0 0.1f
M685 t269 nw44 vdd vdd pch w=2u l=180n
M686 nw74 nw46 t269 vdd pch w=2u l=180n
Cnw74 nw74 0 2f
CT270 t270 0 0.1f
M687 t270 nw48 vdd vdd pch w=2u l=180n
M688 t270 nw52 vdd vdd pch w=2u l=180n
CT271 t271 0 0.1f
M689 t270 nw48 t271 0 nch w=1u l=180n
M690 t271 nw52 0 0 nch w=1u l=180n
M691 nw75 t270 vdd vdd pch w=2u l=180n
M692 nw75 t270 0 0 nch w=1u l=180n
Cnw75 nw75 0 2f
CT272 t272 0 0.1f
M693 t272 nw52 0 0 nch w=1u l=180n
M694 t272 nw58 0 0 nch w=1u l=180n
CT273 t273 0 0.1f
M695 t273 nw52 vdd vdd pch w=2u l=180n
M696 t272 nw58 t273 vdd pch w=2u l=180n
M697 nw76 t272 vdd vdd pch w=2u l=180n
M698 nw76 t272 0 0 nch w=1u l=180n
Cnw76 nw76 0 2f
CT274 t274 0 0.1f
CT275 t275 0 0.1f
CT276 t276 0 0.1f
M699 t274 nw56 vdd vdd pch w=2u l=180n
M700 t274 nw64 vdd vdd pch w=2u l=180n
CT277 t277 0 0.1f
M701 t274 nw56 t277 0 nch w=1u l=180n
M702 t277 nw64 0 0 nch w=1u l=180n
M703 t275 nw56 vdd vdd pch w=2u l=180n
M704 t275 t274 vdd vdd pch w=2u l=180n
CT278 t278 0 0.1f
M705 t275 nw56 t278 0 nch w=1u l=180n
M706 t278 t274 0 0 nch w=1u l=180n
M707 t276 nw64 vdd vdd pch w=2u l=180n
M708 t276 t274 vdd vdd pch w=2u l=180n
CT279 t279 0 0.1f
M709 t276 nw64 t279 0 nch w=1u l=180n
M710 t279 t274 0 0 nch w=1u l=180n
M711 nw77 t275 vdd vdd pch w=2u l=180n
M712 nw77 t276 vdd vdd pch w=2u l=180n
CT280 t280 0 0.1f
M713 nw77 t275 t280 0 nch w=1u l=180n
M714 t280 t276 0 0 nch w=1u l=180n
Cnw77 nw77 0 2f
M715 nw78 nw60 vdd vdd pch w=2u l=180n
M716 nw78 nw70 vdd vdd pch w=2u l=180n
CT281 t281 0 0.1f
M717 nw78 nw60 t281 0 nch w=1u l=180n
M718 t281 nw70 0 0 nch w=1u l=180n
Cnw78 nw78 0 2f
M719 nw79 nw64 0 0 nch w=1u l=180n
M720 nw79 nw76 0 0 nch w=1u l=180n
CT282 t282 0 0.1f
M721 t282 nw64 vdd vdd pch w=2u l=180n
M722 nw79 nw76 t282 vdd pch w=2u l=180n
Cnw79 nw79 0 2f
CT283 t283 0 0.1f
M723 t283 nw68 vdd vdd pch w=2u l=180n
M724 t283 nq2 vdd vdd pch w=2u l=180n
CT284 t284 0 0.1f
M725 t283 nw68 t284 0 nch w=1u l=180n
M726 t284 nq2 0 0 nch w=1u l=180n
M727 nw80 t283 vdd vdd pch w=2u l=180n
M728 nw80 t283 0 0 nch w=1u l=180n
Cnw80 nw80 0 2f
CT285 t285 0 0.1f
M729 t285 nw72 0 0 nch w=1u l=180n
M730 t285 nq7 0 0 nch w=1u l=180n
CT286 t286 0 0.1f
M731 t286 nw72 vdd vdd pch w=2u l=180n
M732 t285 nq7 t286 vdd pch w=2u l=180n
M733 nw81 t285 vdd vdd pch w=2u l=180n
M734 nw81 t285 0 0 nch w=1u l=180n
Cnw81 nw81 0 2f
CT287 t287 0 0.1f
CT288 t288 0 0.1f
CT289 t289 0 0.1f
M735 t287 nw76 vdd vdd pch w=2u l=180n
M736 t287 nq12 vdd vdd pch w=2u l=180n
CT290 t290 0 0.1f
M737 t287 nw76 t290 0 nch w=1u l=180n
M738 t290 nq12 0 0 nch w=1u l=180n
M739 t288 nw76 vdd vdd pch w=2u l=180n
M740 t288 t287 vdd vdd pch w=2u l=180n
CT291 t291 0 0.1f
M741 t288 nw76 t291 0 nch w=1u l=180n
M742 t291 t287 0 0 nch w=1u l=180n
M743 t289 nq12 vdd vdd pch w=2u l=180n
M744 t289 t287 vdd vdd pch w=2u l=180n
CT292 t292 0 0.1f
M745 t289 nq12 t292 0 nch w=1u l=180n
M746 t292 t287 0 0 nch w=1u l=180n
M747 nw82 t288 vdd vdd pch w=2u l=180n
M748 nw82 t289 vdd vdd pch w=2u l=180n
CT293 t293 0 0.1f
M749 nw82 t288 t293 0 nch w=1u l=180n
M750 t293 t289 0 0 nch w=1u l=180n
Cnw82 nw82 0 2f
M751 nw83 nw80 vdd vdd pch w=2u l=180n
M752 nw83 nq17 vdd vdd pch w=2u l=180n
CT294 t294 0 0.1f
M753 nw83 nw80 t294 0 nch w=1u l=180n
M754 t294 nq17 0 0 nch w=1u l=180n
Cnw83 nw83 0 2f
M755 nw84 nq0 0 0 nch w=1u l=180n
M756 nw84 ni1 0 0 nch w=1u l=180n
CT295 t295 0 0.1f
M757 t295 nq0 vdd vdd pch w=2u l=180n
M758 nw84 ni1 t295 vdd pch w=2u l=180n
Cnw84 nw84 0 2f
CT296 t296 0 0.1f
M759 t296 nq3 vdd vdd pch w=2u l=180n
M760 t296 ni6 vdd vdd pch w=2u l=180n
CT297 t297 0 0.1f
M761 t296 nq3 t297 0 nch w=1u l=180n
M762 t297 ni6 0 0 nch w=1u l=180n
M763 nw85 t296 vdd vdd pch w=2u l=180n
M764 nw85 t296 0 0 nch w=1u l=180n
Cnw85 nw85 0 2f
CT298 t298 0 0.1f
M765 t298 nq6 0 0 nch w=1u l=180n
M766 t298 nw44 0 0 nch w=1u l=180n
CT299 t299 0 0.1f
M767 t299 nq6 vdd vdd pch w=2u l=180n
M768 t298 nw44 t299 vdd pch w=2u l=180n
M769 nw86 t298 vdd vdd pch w=2u l=180n
M770 nw86 t298 0 0 nch w=1u l=180n
Cnw86 nw86 0 2f
CT300 t300 0 0.1f
CT301 t301 0 0.1f
CT302 t302 0 0.1f
M771 t300 nq9 vdd vdd pch w=2u l=180n
M772 t300 nw49 vdd vdd pch w=2u l=180n
CT303 t303 0 0.1f
M773 t300 nq9 t303 0 nch w=1u l=180n
M774 t303 nw49 0 0 nch w=1u l=180n
M775 t301 nq9 vdd vdd pch w=2u l=180n
M776 t301 t300 vdd vdd pch w=2u l=180n
CT304 t304 0 0.1f
M777 t301 nq9 t304 0 nch w=1u l=180n
M778 t304 t300 0 0 nch w=1u l=180n
M779 t302 nw49 vdd vdd pch w=2u l=180n
M780 t302 t300 vdd vdd pch w=2u l=180n
CT305 t305 0 0.1f
M781 t302 nw49 t305 0 nch w=1u l=180n
M782 t305 t300 0 0 nch w=1u l=180n
M783 nw87 t301 vdd vdd pch w=2u l=180n
M784 nw87 t302 vdd vdd pch w=2u l=180n
CT306 t306 0 0.1f
M785 nw87 t301 t306 0 nch w=1u l=180n
M786 t306 t302 0 0 nch w=1u l=180n
Cnw87 nw87 0 2f
M787 nw88 nq12 vdd vdd pch w=2u l=180n
M788 nw88 nw54 vdd vdd pch w=2u l=180n
CT307 t307 0 0.1f
M789 nw88 nq12 t307 0 nch w=1u l=180n
M790 t307 nw54 0 0 nch w=1u l=180n
Cnw88 nw88 0 2f
M791 nw89 nq15 0 0 nch w=1u l=180n
M792 nw89 nw59 0 0 nch w=1u l=180n
CT308 t308 0 0.1f
M793 t308 nq15 vdd vdd pch w=2u l=180n
M794 nw89 nw59 t308 vdd pch w=2u l=180n
Cnw89 nw89 0 2f
CT309 t309 0 0.1f
M795 t309 nq18 vdd vdd pch w=2u l=180n
M796 t309 nw64 vdd vdd pch w=2u l=180n
CT310 t310 0 0.1f
M797 t309 nq18 t310 0 nch w=1u l=180n
M798 t310 nw64 0 0 nch w=1u l=180n
M799 nw90 t309 vdd vdd pch w=2u l=180n
M800 nw90 t309 0 0 nch w=1u l=180n
Cnw90 nw90 0 2f
CT311 t311 0 0.1f
M801 t311 ni0 0 0 nch w=1u l=180n
M802 t311 nw69 0 0 nch w=1u l=180n
CT312 t312 0 0.1f
M803 t312 ni0 vdd vdd pch w=2u l=180n
M804 t311 nw69 t312 vdd pch w=2u l=180n
M805 nw91 t311 vdd vdd pch w=2u l=180n
M806 nw91 t311 0 0 nch w=1u l=180n
Cnw91 nw91 0 2f
CT313 t313 0 0.1f
CT314 t314 0 0.1f
CT315 t315 0 0.1f
M807 t313 ni3 vdd vdd pch w=2u l=180n
M808 t313 nw74 vdd vdd pch w=2u l=180n
CT316 t316 0 0.1f
M809 t313 ni3 t316 0 nch w=1u l=180n
M810 t316 nw74 0 0 nch w=1u l=180n
M811 t314 ni3 vdd vdd pch w=2u l=180n
M812 t314 t313 vdd vdd pch w=2u l=180n
CT317 t317 0 0.1f
M813 t314 ni3 t317 0 nch w=1u l=180n
M814 t317 t313 0 0 nch w=1u l=180n
M815 t315 nw74 vdd vdd pch w=2u l=180n
M816 t315 t313 vdd vdd pch w=2u l=180n
CT318 t318 0 0.1f
M817 t315 nw74 t318 0 nch w=1u l=180n
M818 t318 t313 0 0 nch w=1u l=180n
M819 nw92 t314 vdd vdd pch w=2u l=180n
M820 nw92 t315 vdd vdd pch w=2u l=180n
CT319 t319 0 0.1f
M821 nw92 t314 t319 0 nch w=1u l=180n
M822 t319 t315 0 0 nch w=1u l=180n
Cnw92 nw92 0 2f
M823 nw93 ni6 vdd vdd pch w=2u l=180n
M824 nw93 nw79 vdd vdd pch w=2u l=180n
CT320 t320 0 0.1f
M825 nw93 ni6 t320 0 nch w=1u l=180n
M826 t320 nw79 0 0 nch w=1u l=180n
Cnw93 nw93 0 2f
M827 nw94 ni9 0 0 nch w=1u l=180n
M828 nw94 nw84 0 0 nch w=1u l=180n
CT321 t321 0 0.1f
M829 t321 ni9 vdd vdd pch w=2u l=180n
M830 nw94 nw84 t321 vdd pch w=2u l=180n
Cnw94 nw94 0 2f
CT322 t322 0 0.1f
M831 t322 nw45 vdd vdd pch w=2u l=180n
M832 t322 nw89 vdd vdd pch w=2u l=180n
CT323 t323 0 0.1f
M833 t322 nw45 t323 0 nch w=1u l=180n
M834 t323 nw89 0 0 nch w=1u l=180n
M835 nw95 t322 vdd vdd pch w=2u l=180n
M836 nw95 t322 0 0 nch w=1u l=180n
Cnw95 nw95 0 2f
CT324 t324 0 0.1f
M837 t324 nw48 0 0 nch w=1u l=180n
M838 t324 nw94 0 0 nch w=1u l=180n
CT325 t325 0 0.1f
M839 t325 nw48 vdd vdd pch w=2u l=180n
M840 t324 nw94 t325 vdd pch w=2u l=180n
M841 nw96 t324 vdd vdd pch w=2u l=180n
M842 nw96 t324 0 0 nch w=1u l=180n
Cnw96 nw96 0 2f
CT326 t326 0 0.1f
CT327 t327 0 0.1f
CT328 t328 0 0.1f
M843 t326 nw51 vdd vdd pch w=2u l=180n
M844 t326 nq2 vdd vdd pch w=2u l=180n
CT329 t329 0 0.1f
M845 t326 nw51 t329 0 nch w=1u l=180n
M846 t329 nq2 0 0 nch w=1u l=180n
M847 t327 nw51 vdd vdd pch w=2u l=180n
M848 t327 t326 vdd vdd pch w=2u l=180n
CT330 t330 0 0.1f
M849 t327 nw51 t330 0 nch w=1u l=180n
M850 t330 t326 0 0 nch w=1u l=180n
M851 t328 nq2 vdd vdd pch w=2u l=180n
M852 t328 t326 vdd vdd pch w=2u l=180n
CT331 t331 0 0.1f
M853 t328 nq2 t331 0 nch w=1u l=180n
M854 t331 t326 0 0 nch w=1u l=180n
M855 nw97 t327 vdd vdd pch w=2u l=180n
M856 nw97 t328 vdd vdd pch w=2u l=180n
CT332 t332 0 0.1f
M857 nw97 t327 t332 0 nch w=1u l=180n
M858 t332 t328 0 0 nch w=1u l=180n
Cnw97 nw97 0 2f
M859 nw98 nw54 vdd vdd pch w=2u l=180n
M860 nw98 nq6 vdd vdd pch w=2u l=180n
CT333 t333 0 0.1f
M861 nw98 nw54 t333 0 nch w=1u l=180n
M862 t333 nq6 0 0 nch w=1u l=180n
Cnw98 nw98 0 2f
M863 nw99 nw57 0 0 nch w=1u l=180n
M864 nw99 nq10 0 0 nch w=1u l=180n
CT334 t334 0 0.1f
M865 t334 nw57 vdd vdd pch w=2u l=180n
M866 nw99 nq10 t334 vdd pch w=2u l=180n
Cnw99 nw99 0 2f
CT335 t335 0 0.1f
M867 t335 nw60 vdd vdd pch w=2u l=180n
M868 t335 nq14 vdd vdd pch w=2u l=180n
CT336 t336 0 0.1f
M869 t335 nw60 t336 0 nch w=1u l=180n
M870 t336 nq14 0 0 nch w=1u l=180n
M871 nw100 t335 vdd vdd pch w=2u l=180n
M872 nw100 t335 0 0 nch w=1u l=180n
Cnw100 nw100 0 2f
CT337 t337 0 0.1f
M873 t337 nw63 0 0 nch w=1u l=180n
M874 t337 nq18 0 0 nch w=1u l=180n
CT338 t338 0 0.1f
M875 t338 nw63 vdd vdd pch w=2u l=180n
M876 t337 nq18 t338 vdd pch w=2u l=180n
M877 nw101 t337 vdd vdd pch w=2u l=180n
M878 nw101 t337 0 0 nch w=1u l=180n
Cnw101 nw101 0 2f
CT339 t339 0 0.1f
CT340 t340 0 0.1f
CT341 t341 0 0.1f
M879 t339 nw66 vdd vdd pch w=2u l=180n
M880 t339 ni1 vdd vdd pch w=2u l=180n
CT342 t342 0 0.1f
M881 t339 nw66 t342 0 nch w=1u l=180n
M882 t342 ni1 0 0 nch w=1u l=180n
M883 t340 nw66 vdd vdd pch w=2u l=180n
M884 t340 t339 vdd vdd pch w=2u l=180n
CT343 t343 0 0.1f
M885 t340 nw66 t343 0 nch w=1u l=180n
M886 t343 t339 0 0 nch w=1u l=180n
M887 t341 ni1 vdd vdd pch w=2u l=180n
M888 t341 t339 vdd vdd pch w=2u l=180n
CT344 t344 0 0.1f
M889 t341 ni1 t344 0 nch w=1u l=180n
M890 t344 t339 0 0 nch w=1u l=180n
M891 nw102 t340 vdd vdd pch w=2u l=180n
M892 nw102 t341 vdd vdd pch w=2u l=180n
CT345 t345 0 0.1f
M893 nw102 t340 t345 0 nch w=1u l=180n
M894 t345 t341 0 0 nch w=1u l=180n
Cnw102 nw102 0 2f
M895 nw103 nw69 vdd vdd pch w=2u l=180n
M896 nw103 ni5 vdd vdd pch w=2u l=180n
CT346 t346 0 0.1f
M897 nw103 nw69 t346 0 nch w=1u l=180n
M898 t346 ni5 0 0 nch w=1u l=180n
Cnw103 nw103 0 2f
M899 nw104 nw72 0 0 nch w=1u l=180n
M900 nw104 ni9 0 0 nch w=1u l=180n
CT347 t347 0 0.1f
M901 t347 nw72 vdd vdd pch w=2u l=180n
M902 nw104 ni9 t347 vdd pch w=2u l=180n
Cnw104 nw104 0 2f
CT348 t348 0 0.1f
M903 t348 nw75 vdd vdd pch w=2u l=180n
M904 t348 nw46 vdd vdd pch w=2u l=180n
CT349 t349 0 0.1f
M905 t348 nw75 t349 0 nch w=1u l=180n
M906 t349 nw46 0 0 nch w=1u l=180n
M907 nw105 t348 vdd vdd pch w=2u l=180n
M908 nw105 t348 0 0 nch w=1u l=180n
Cnw105 nw105 0 2f
CT350 t350 0 0.1f
M909 t350 nw78 0 0 nch w=1u l=180n
M910 t350 nw50 0 0 nch w=1u l=180n
CT351 t351 0 0.1f
M911 t351 nw78 vdd vdd pch w=2u l=180n
M912 t350 nw50 t351 vdd pch w=2u l=180n
M913 nw106 t350 vdd vdd pch w=2u l=180n
M914 nw106 t350 0 0 nch w=1u l=180n
Cnw106 nw106 0 2f
CT352 t352 0 0.1f
CT353 t353 0 0.1f
CT354 t354 0 0.1f
M915 t352 nw81 vdd vdd pch w=2u l=180n
M916 t352 nw54 vdd vdd pch w=2u l=180n
CT355 t355 0 0.1f
M917 t352 nw81 t355 0 nch w=1u l=180n
M918 t355 nw54 0 0 nch w=1u l=180n
M919 t353 nw81 vdd vdd pch w=2u l=180n
M920 t353 t352 vdd vdd pch w=2u l=180n
CT356 t356 0 0.1f
M921 t353 nw81 t356 0 nch w=1u l=180n
M922 t356 t352 0 0 nch w=1u l=180n
M923 t354 nw54 vdd vdd pch w=2u l=180n
M924 t354 t352 vdd vdd pch w=2u l=180n
CT357 t357 0 0.1f
M925 t354 nw54 t357 0 nch w=1u l=180n
M926 t357 t352 0 0 nch w=1u l=180n
M927 nw107 t353 vdd vdd pch w=2u l=180n
M928 nw107 t354 vdd vdd pch w=2u l=180n
CT358 t358 0 0.1f
M929 nw107 t353 t358 0 nch w=1u l=180n
M930 t358 t354 0 0 nch w=1u l=180n
Cnw107 nw107 0 2f
M931 nw108 nw84 vdd vdd pch w=2u l=180n
M932 nw108 nw58 vdd vdd pch w=2u l=180n
CT359 t359 0 0.1f
M933 nw108 nw84 t359 0 nch w=1u l=180n
M934 t359 nw58 0 0 nch w=1u l=180n
Cnw108 nw108 0 2f
M935 nw109 nw87 0 0 nch w=1u l=180n
M936 nw109 nw62 0 0 nch w=1u l=180n
CT360 t360 0 0.1f
M937 t360 nw87 vdd vdd pch w=2u l=180n
M938 nw109 nw62 t360 vdd pch w=2u l=180n
Cnw109 nw109 0 2f
CT361 t361 0 0.1f
M939 t361 nw90 vdd vdd pch w=2u l=180n
M940 t361 nw66 vdd vdd pch w=2u l=180n
CT362 t362 0 0.1f
M941 t361 nw90 t362 0 nch w=1u l=180n
M942 t362 nw66 0 0 nch w=1u l=180n
M943 nw110 t361 vdd vdd pch w=2u l=180n
M944 nw110 t361 0 0 nch w=1u l=180n
Cnw110 nw110 0 2f
CT363 t363 0 0.1f
M945 t363 nw93 0 0 nch w=1u l=180n
M946 t363 nw70 0 0 nch w=1u l=180n
CT364 t364 0 0.1f
M947 t364 nw93 vdd vdd pch w=2u l=180n
M948 t363 nw70 t364 vdd pch w=2u l=180n
M949 nw111 t363 vdd vdd pch w=2u l=180n
M950 nw111 t363 0 0 nch w=1u l=180n
Cnw111 nw111 0 2f
CT365 t365 0 0.1f
CT366 t366 0 0.1f
CT367 t367 0 0.1f
M951 t365 nw96 vdd vdd pch w=2u l=180n
M952 t365 nw74 vdd vdd pch w=2u l=180n
CT368 t368 0 0.1f
M953 t365 nw96 t368 0 nch w=1u l=180n
M954 t368 nw74 0 0 nch w=1u l=180n
M955 t366 nw96 vdd vdd pch w=2u l=180n
M956 t366 t365 vdd vdd pch w=2u l=180n
CT369 t369 0 0.1f
M957 t366 nw96 t369 0 nch w=1u l=180n
M958 t369 t365 0 0 nch w=1u l=180n
M959 t367 nw74 vdd vdd pch w=2u l=180n
M960 t367 t365 vdd vdd pch w=2u l=180n
CT370 t370 0 0.1f
M961 t367 nw74 t370 0 nch w=1u l=180n
M962 t370 t365 0 0 nch w=1u l=180n
M963 nw112 t366 vdd vdd pch w=2u l=180n
M964 nw112 t367 vdd vdd pch w=2u l=180n
CT371 t371 0 0.1f
M965 nw112 t366 t371 0 nch w=1u l=180n
M966 t371 t367 0 0 nch w=1u l=180n
Cnw112 nw112 0 2f
M967 nw113 nw99 vdd vdd pch w=2u l=180n
M968 nw113 nw78 vdd vdd pch w=2u l=180n
CT372 t372 0 0.1f
M969 nw113 nw99 t372 0 nch w=1u l=180n
M970 t372 nw78 0 0 nch w=1u l=180n
Cnw113 nw113 0 2f
M971 nw114 nw102 0 0 nch w=1u l=180n
M972 nw114 nw82 0 0 nch w=1u l=180n
CT373 t373 0 0.1f
M973 t373 nw102 vdd vdd pch w=2u l=180n
M974 nw114 nw82 t373 vdd pch w=2u l=180n
Cnw114 nw114 0 2f
CT374 t374 0 0.1f
M975 t374 nw105 vdd vdd pch w=2u l=180n
M976 t374 nw86 vdd vdd pch w=2u l=180n
CT375 t375 0 0.1f
M977 t374 nw105 t375 0 nch w=1u l=180n
M978 t375 nw86 0 0 nch w=1u l=180n
M979 nw115 t374 vdd vdd pch w=2u l=180n
M980 nw115 t374 0 0 nch w=1u l=180n
Cnw115 nw115 0 2f
CT376 t376 0 0.1f
M981 t376 nw108 0 0 nch w=1u l=180n
M982 t376 nw90 0 0 nch w=1u l=180n
CT377 t377 0 0.1f
M983 t377 nw108 vdd vdd pch w=2u l=180n
M984 t376 nw90 t377 vdd pch w=2u l=180n
M985 nw116 t376 vdd vdd pch w=2u l=180n
M986 nw116 t376 0 0 nch w=1u l=180n
Cnw116 nw116 0 2f
CT378 t378 0 0.1f
CT379 t379 0 0.1f
CT380 t380 0 0.1f
M987 t378 nw111 vdd vdd pch w=2u l=180n
M988 t378 nw94 vdd vdd pch w=2u l=180n
CT381 t381 0 0.1f
M989 t378 nw111 t381 0 nch w=1u l=180n
M990 t381 nw94 0 0 nch w=1u l=180n
M991 t379 nw111 vdd vdd pch w=2u l=180n
M992 t379 t378 vdd vdd pch w=2u l=180n
CT382 t382 0 0.1f
M993 t379 nw111 t382 0 nch w=1u l=180n
M994 t382 t378 0 0 nch w=1u l=180n
M995 t380 nw94 vdd vdd pch w=2u l=180n
M996 t380 t378 vdd vdd pch w=2u l=180n
CT383 t383 0 0.1f
M997 t380 nw94 t383 0 nch w=1u l=180n
M998 t383 t378 0 0 nch w=1u l=180n
M999 nw117 t379 vdd vdd pch w=2u l=180n
M1000 nw117 t380 vdd vdd pch w=2u l=180n
CT384 t384 0 0.1f
M1001 nw117 t379 t384 0 nch w=1u l=180n
M1002 t384 t380 0 0 nch w=1u l=180n
Cnw117 nw117 0 2f
M1003 nw118 nw114 vdd vdd pch w=2u l=180n
M1004 nw118 nw98 vdd vdd pch w=2u l=180n
CT385 t385 0 0.1f
M1005 nw118 nw114 t385 0 nch w=1u l=180n
M1006 t385 nw98 0 0 nch w=1u l=180n
Cnw118 nw118 0 2f
M1007 nw119 nw117 0 0 nch w=1u l=180n
M1008 nw119 nw102 0 0 nch w=1u l=180n
CT386 t386 0 0.1f
M1009 t386 nw117 vdd vdd pch w=2u l=180n
M1010 nw119 nw102 t386 vdd pch w=2u l=180n
Cnw119 nw119 0 2f
CT387 t387 0 0.1f
M1011 t387 nq0 vdd vdd pch w=2u l=180n
M1012 t387 nw106 vdd vdd pch w=2u l=180n
CT388 t388 0 0.1f
M1013 t387 nq0 t388 0 nch w=1u l=180n
M1014 t388 nw106 0 0 nch w=1u l=180n
M1015 nw120 t387 vdd vdd pch w=2u l=180n
M1016 nw120 t387 0 0 nch w=1u l=180n
Cnw120 nw120 0 2f
CT389 t389 0 0.1f
M1017 t389 nq2 0 0 nch w=1u l=180n
M1018 t389 nw110 0 0 nch w=1u l=180n
CT390 t390 0 0.1f
M1019 t390 nq2 vdd vdd pch w=2u l=180n
M1020 t389 nw110 t390 vdd pch w=2u l=180n
M1021 nw121 t389 vdd vdd pch w=2u l=180n
M1022 nw121 t389 0 0 nch w=1u l=180n
Cnw121 nw121 0 2f
CT391 t391 0 0.1f
CT392 t392 0 0.1f
CT393 t393 0 0.1f
M1023 t391 nq4 vdd vdd pch w=2u l=180n
M1024 t391 nw114 vdd vdd pch w=2u l=180n
CT394 t394 0 0.1f
M1025 t391 nq4 t394 0 nch w=1u l=180n
M1026 t394 nw114 0 0 nch w=1u l=180n
M1027 t392 nq4 vdd vdd pch w=2u l=180n
M1028 t392 t391 vdd vdd pch w=2u l=180n
CT395 t395 0 0.1f
M1029 t392 nq4 t395 0 nch w=1u l=180n
M1030 t395 t391 0 0 nch w=1u l=180n
M1031 t393 nw114 vdd vdd pch w=2u l=180n
M1032 t393 t391 vdd vdd pch w=2u l=180n
CT396 t396 0 0.1f
M1033 t393 nw114 t396 0 nch w=1u l=180n
M1034 t396 t391 0 0 nch w=1u l=180n
M1035 nw122 t392 vdd vdd pch w=2u l=180n
M1036 nw122 t393 vdd vdd pch w=2u l=180n
CT397 t397 0 0.1f
M1037 nw122 t392 t397 0 nch w=1u l=180n
M1038 t397 t393 0 0 nch w=1u l=180n
Cnw122 nw122 0 2f
M1039 nw123 nq6 vdd vdd pch w=2u l=180n
M1040 nw123 nw118 vdd vdd pch w=2u l=180n
CT398 t398 0 0.1f
M1041 nw123 nq6 t398 0 nch w=1u l=180n
M1042 t398 nw118 0 0 nch w=1u l=180n
Cnw123 nw123 0 2f
M1043 nw124 nq8 0 0 nch w=1u l=180n
M1044 nw124 nw122 0 0 nch w=1u l=180n
CT399 t399 0 0.1f
M1045 t399 nq8 vdd vdd pch w=2u l=180n
M1046 nw124 nw122 t399 vdd pch w=2u l=180n
Cnw124 nw124 0 2f
CT400 t400 0 0.1f
M1047 t400 nq10 vdd vdd pch w=2u l=180n
M1048 t400 nq1 vdd vdd pch w=2u l=180n
CT401 t401 0 0.1f
M1049 t400 nq10 t401 0 nch w=1u l=180n
M1050 t401 nq1 0 0 nch w=1u l=180n
M1051 nw125 t400 vdd vdd pch w=2u l=180n
M1052 nw125 t400 0 0 nch w=1u l=180n
Cnw125 nw125 0 2f
CT402 t402 0 0.1f
M1053 t402 nq12 0 0 nch w=1u l=180n
M1054 t402 nq4 0 0 nch w=1u l=180n
CT403 t403 0 0.1f
M1055 t403 nq12 vdd vdd pch w=2u l=180n
M1056 t402 nq4 t403 vdd pch w=2u l=180n
M1057 nw126 t402 vdd vdd pch w=2u l=180n
M1058 nw126 t402 0 0 nch w=1u l=180n
Cnw126 nw126 0 2f
CT404 t404 0 0.1f
CT405 t405 0 0.1f
CT406 t406 0 0.1f
M1059 t404 nq14 vdd vdd pch w=2u l=180n
M1060 t404 nq7 vdd vdd pch w=2u l=180n
CT407 t407 0 0.1f
M1061 t404 nq14 t407 0 nch w=1u l=180n
M1062 t407 nq7 0 0 nch w=1u l=180n
M1063 t405 nq14 vdd vdd pch w=2u l=180n
M1064 t405 t404 vdd vdd pch w=2u l=180n
CT408 t408 0 0.1f
M1065 t405 nq14 t408 0 nch w=1u l=180n
M1066 t408 t404 0 0 nch w=1u l=180n
M1067 t406 nq7 vdd vdd pch w=2u l=180n
M1068 t406 t404 vdd vdd pch w=2u l=180n
CT409 t409 0 0.1f
M1069 t406 nq7 t409 0 nch w=1u l=180n
M1070 t409 t404 0 0 nch w=1u l=180n
M1071 nw127 t405 vdd vdd pch w=2u l=180n
M1072 nw127 t406 vdd vdd pch w=2u l=180n
CT410 t410 0 0.1f
M1073 nw127 t405 t410 0 nch w=1u l=180n
M1074 t410 t406 0 0 nch w=1u l=180n
Cnw127 nw127 0 2f
M1075 nw128 nq16 vdd vdd pch w=2u l=180n
M1076 nw128 nq10 vdd vdd pch w=2u l=180n
CT411 t411 0 0.1f
M1077 nw128 nq16 t411 0 nch w=1u l=180n
M1078 t411 nq10 0 0 nch w=1u l=180n
Cnw128 nw128 0 2f
M1079 nw129 nq18 0 0 nch w=1u l=180n
M1080 nw129 nq13 0 0 nch w=1u l=180n
CT412 t412 0 0.1f
M1081 t412 nq18 vdd vdd pch w=2u l=180n
M1082 nw129 nq13 t412 vdd pch w=2u l=180n
Cnw129 nw129 0 2f
CT413 t413 0 0.1f
M1083 t413 nq20 vdd vdd pch w=2u l=180n
M1084 t413 nq16 vdd vdd pch w=2u l=180n
CT414 t414 0 0.1f
M1085 t413 nq20 t414 0 nch w=1u l=180n
M1086 t414 nq16 0 0 nch w=1u l=180n
M1087 nw130 t413 vdd vdd pch w=2u l=180n
M1088 nw130 t413 0 0 nch w=1u l=180n
Cnw130 nw130 0 2f
CT415 t415 0 0.1f
M1089 t415 ni1 0 0 nch w=1u l=180n
M1090 t415 nq19 0 0 nch w=1u l=180n
CT416 t416 0 0.1f
M1091 t416 ni1 vdd vdd pch w=2u l=180n
M1092 t415 nq19 t416 vdd pch w=2u l=180n
M1093 nw131 t415 vdd vdd pch w=2u l=180n
M1094 nw131 t415 0 0 nch w=1u l=180n
Cnw131 nw131 0 2f
CT417 t417 0 0.1f
CT418 t418 0 0.1f
CT419 t419 0 0.1f
M1095 t417 ni3 vdd vdd pch w=2u l=180n
M1096 t417 ni1 vdd vdd pch w=2u l=180n
CT420 t420 0 0.1f
M1097 t417 ni3 t420 0 nch w=1u l=180n
M1098 t420 ni1 0 0 nch w=1u l=180n
M1099 t418 ni3 vdd vdd pch w=2u l=180n
M1100 t418 t417 vdd vdd pch w=2u l=180n
CT421 t421 0 0.1f
M1101 t418 ni3 t421 0 nch w=1u l=180n
M1102 t421 t417 0 0 nch w=1u l=180n
M1103 t419 ni1 vdd vdd pch w=2u l=180n
M1104 t419 t417 vdd vdd pch w=2u l=180n
CT422 t422 0 0.1f
M1105 t419 ni1 t422 0 nch w=1u l=180n
M1106 t422 t417 0 0 nch w=1u l=180n
M1107 nw132 t418 vdd vdd pch w=2u l=180n
M1108 nw132 t419 vdd vdd pch w=2u l=180n
CT423 t423 0 0.1f
M1109 nw132 t418 t423 0 nch w=1u l=180n
M1110 t423 t419 0 0 nch w=1u l=180n
Cnw132 nw132 0 2f
M1111 nw133 ni5 vdd vdd pch w=2u l=180n
M1112 nw133 ni4 vdd vdd pch w=2u l=180n
CT424 t424 0 0.1f
M1113 nw133 ni5 t424 0 nch w=1u l=180n
M1114 t424 ni4 0 0 nch w=1u l=180n
Cnw133 nw133 0 2f
M1115 nw134 ni7 0 0 nch w=1u l=180n
M1116 nw134 nw102 0 0 nch w=1u l=180n
CT425 t425 0 0.1f
M1117 t425 ni7 vdd vdd pch w=2u l=180n
M1118 nw134 nw102 t425 vdd pch w=2u l=180n
Cnw134 nw134 0 2f
CT426 t426 0 0.1f
M1119 t426 ni9 vdd vdd pch w=2u l=180n
M1120 t426 nw43 vdd vdd pch w=2u l=180n
CT427 t427 0 0.1f
M1121 t426 ni9 t427 0 nch w=1u l=180n
M1122 t427 nw43 0 0 nch w=1u l=180n
M1123 nw135 t426 vdd vdd pch w=2u l=180n
M1124 nw135 t426 0 0 nch w=1u l=180n
Cnw135 nw135 0 2f
CT428 t428 0 0.1f
M1125 t428 nw44 0 0 nch w=1u l=180n
M1126 t428 nw46 0 0 nch w=1u l=180n
CT429 t429 0 0.1f
M1127 t429 nw44 vdd vdd pch w=2u l=180n
M1128 t428 nw46 t429 vdd pch w=2u l=180n
M1129 nw136 t428 vdd vdd pch w=2u l=180n
M1130 nw136 t428 0 0 nch w=1u l=180n
Cnw136 nw136 0 2f
CT430 t430 0 0.1f
CT431 t431 0 0.1f
CT432 t432 0 0.1f
M1131 t430 nw46 vdd vdd pch w=2u l=180n
M1132 t430 nw49 vdd vdd pch w=2u l=180n
CT433 t433 0 0.1f
M1133 t430 nw46 t433 0 nch w=1u l=180n
M1134 t433 nw49 0 0 nch w=1u l=180n
M1135 t431 nw46 vdd vdd pch w=2u l=180n
M1136 t431 t430 vdd vdd pch w=2u l=180n
CT434 t434 0 0.1f
M1137 t431 nw46 t434 0 nch w=1u l=180n
M1138 t434 t430 0 0 nch w=1u l=180n
M1139 t432 nw49 vdd vdd pch w=2u l=180n
M1140 t432 t430 vdd vdd pch w=2u l=180n
CT435 t435 0 0.1f
M1141 t432 nw49 t435 0 nch w=1u l=180n
M1142 t435 t430 0 0 nch w=1u l=180n
M1143 nw137 t431 vdd vdd pch w=2u l=180n
M1144 nw137 t432 vdd vdd pch w=2u l=180n
CT436 t436 0 0.1f
M1145 nw137 t431 t436 0 nch w=1u l=180n
M1146 t436 t432 0 0 nch w=1u l=180n
Cnw137 nw137 0 2f
M1147 nw138 nw48 vdd vdd pch w=2u l=180n
M1148 nw138 nw52 vdd vdd pch w=2u l=180n
CT437 t437 0 0.1f
M1149 nw138 nw48 t437 0 nch w=1u l=180n
M1150 t437 nw52 0 0 nch w=1u l=180n
Cnw138 nw138 0 2f
M1151 nw139 nw50 0 0 nch w=1u l=180n
M1152 nw139 nw55 0 0 nch w=1u l=180n
CT438 t438 0 0.1f
M1153 t438 nw50 vdd vdd pch w=2u l=180n
M1154 nw139 nw55 t438 vdd pch w=2u l=180n
Cnw139 nw139 0 2f
CT439 t439 0 0.1f
M1155 t439 nw52 vdd vdd pch w=2u l=180n
M1156 t439 nw58 vdd vdd pch w=2u l=180n
CT440 t440 0 0.1f
M1157 t439 nw52 t440 0 nch w=1u l=180n
M1158 t440 nw58 0 0 nch w=1u l=180n
M1159 nw140 t439 vdd vdd pch w=2u l=180n
M1160 nw140 t439 0 0 nch w=1u l=180n
Cnw140 nw140 0 2f
CT441 t441 0 0.1f
M1161 t441 nw54 0 0 nch w=1u l=180n
M1162 t441 nw61 0 0 nch w=1u l=180n
CT442 t442 0 0.1f
M1163 t442 nw54 vdd vdd pch w=2u l=180n
M1164 t441 nw61 t442 vdd pch w=2u l=180n
M1165 nw141 t441 vdd vdd pch w=2u l=180n
M1166 nw141 t441 0 0 nch w=1u l=180n
Cnw141 nw141 0 2f
CT443 t443 0 0.1f
CT444 t444 0 0.1f
CT445 t445 0 0.1f
M1167 t443 nw56 vdd vdd pch w=2u l=180n
M1168 t443 nw64 vdd vdd pch w=2u l=180n
CT446 t446 0 0.1f
M1169 t443 nw56 t446 0 nch w=1u l=180n
M1170 t446 nw64 0 0 nch w=1u l=180n
M1171 t444 nw56 vdd vdd pch w=2u l=180n
M1172 t444 t443 vdd vdd pch w=2u l=180n
CT447 t447 0 0.1f
M1173 t444 nw56 t447 0 nch w=1u l=180n
M1174 t447 t443 0 0 nch w=1u l=180n
M1175 t445 nw64 vdd vdd pch w=2u l=180n
M1176 t445 t443 vdd vdd pch w=2u l=180n
CT448 t448 0 0.1f
M1177 t445 nw64 t448 0 nch w=1u l=180n
M1178 t448 t443 0 0 nch w=1u l=180n
M1179 nw142 t444 vdd vdd pch w=2u l=180n
M1180 nw142 t445 vdd vdd pch w=2u l=180n
CT449 t449 0 0.1f
M1181 nw142 t444 t449 0 nch w=1u l=180n
M1182 t449 t445 0 0 nch w=1u l=180n
Cnw142 nw142 0 2f
M1183 nw143 nw58 vdd vdd pch w=2u l=180n
M1184 nw143 nw67 vdd vdd pch w=2u l=180n
CT450 t450 0 0.1f
M1185 nw143 nw58 t450 0 nch w=1u l=180n
M1186 t450 nw67 0 0 nch w=1u l=180n
Cnw143 nw143 0 2f
M1187 nw144 nw60 0 0 nch w=1u l=180n
M1188 nw144 nw70 0 0 nch w=1u l=180n
CT451 t451 0 0.1f
M1189 t451 nw60 vdd vdd pch w=2u l=180n
M1190 nw144 nw70 t451 vdd pch w=2u l=180n
Cnw144 nw144 0 2f
CT452 t452 0 0.1f
M1191 t452 nw62 vdd vdd pch w=2u l=180n
M1192 t452 nw73 vdd vdd pch w=2u l=180n
CT453 t453 0 0.1f
M1193 t452 nw62 t453 0 nch w=1u l=180n
M1194 t453 nw73 0 0 nch w=1u l=180n
M1195 nw145 t452 vdd vdd pch w=2u l=180n
M1196 nw145 t452 0 0 nch w=1u l=180n
Cnw145 nw145 0 2f
CT454 t454 0 0.1f
M1197 t454 nw64 0 0 nch w=1u l=180n
M1198 t454 nw76 0 0 nch w=1u l=180n
CT455 t455 0 0.1f
M1199 t455 nw64 vdd vdd pch w=2u l=180n
M1200 t454 nw76 t455 vdd pch w=2u l=180n
M1201 nw146 t454 vdd vdd pch w=2u l=180n
M1202 nw146 t454 0 0 nch w=1u l=180n
Cnw146 nw146 0 2f
CT456 t456 0 0.1f
CT457 t457 0 0.1f
CT458 t458 0 0.1f
M1203 t456 nw66 vdd vdd pch w=2u l=180n
M1204 t456 nw79 vdd vdd pch w=2u l=180n
CT459 t459 0 0.1f
M1205 t456 nw66 t459 0 nch w=1u l=180n
M1206 t459 nw79 0 0 nch w=1u l=180n
M1207 t457 nw66 vdd vdd pch w=2u l=180n
M1208 t457 t456 vdd vdd pch w=2u l=180n
CT460 t460 0 0.1f
M1209 t457 nw66 t460 0 nch w=1u l=180n
M1210 t460 t456 0 0 nch w=1u l=180n
M1211 t458 nw79 vdd vdd pch w=2u l=180n
M1212 t458 t456 vdd vdd pch w=2u l=180n
CT461 t461 0 0.1f
M1213 t458 nw79 t461 0 nch w=1u l=180n
M1214 t461 t456 0 0 nch w=1u l=180n
M1215 nw147 t457 vdd vdd pch w=2u l=180n
M1216 nw147 t458 vdd vdd pch w=2u l=180n
CT462 t462 0 0.1f
M1217 nw147 t457 t462 0 nch w=1u l=180n
M1218 t462 t458 0 0 nch w=1u l=180n
Cnw147 nw147 0 2f
M1219 nw148 nw68 vdd vdd pch w=2u l=180n
M1220 nw148 nw82 vdd vdd pch w=2u l=180n
CT463 t463 0 0.1f
M1221 nw148 nw68 t463 0 nch w=1u l=180n
M1222 t463 nw82 0 0 nch w=1u l=180n
Cnw148 nw148 0 2f
M1223 nw149 nw70 0 0 nch w=1u l=180n
M1224 nw149 nw85 0 0 nch w=1u l=180n
CT464 t464 0 0.1f
M1225 t464 nw70 vdd vdd pch w=2u l=180n
M1226 nw149 nw85 t464 vdd pch w=2u l=180n
Cnw149 nw149 0 2f
CT465 t465 0 0.1f
M1227 t465 nw72 vdd vdd pch w=2u l=180n
M1228 t465 nw88 vdd vdd pch w=2u l=180n
CT466 t466 0 0.1f
M1229 t465 nw72 t466 0 nch w=1u l=180n
M1230 t466 nw88 0 0 nch w=1u l=180n
M1231 nw150 t465 vdd vdd pch w=2u l=180n
M1232 nw150 t465 0 0 nch w=1u l=180n
Cnw150 nw150 0 2f
CT467 t467 0 0.1f
M1233 t467 nw74 0 0 nch w=1u l=180n
M1234 t467 nw91 0 0 nch w=1u l=180n
CT468 t468 0 0.1f
M1235 t468 nw74 vdd vdd pch w=2u l=180n
M1236 t467 nw91 t468 vdd pch w=2u l=180n
M1237 nw151 t467 vdd vdd pch w=2u l=180n
M1238 nw151 t467 0 0 nch w=1u l=180n
Cnw151 nw151 0 2f
CT469 t469 0 0.1f
CT470 t470 0 0.1f
CT471 t471 0 0.1f
M1239 t469 nw76 vdd vdd pch w=2u l=180n
M1240 t469 nw94 vdd vdd pch w=2u l=180n
CT472 t472 0 0.1f
M1241 t469 nw76 t472 0 nch w=1u l=180n
M1242 t472 nw94 0 0 nch w=1u l=180n
M1243 t470 nw76 vdd vdd pch w=2u l=180n
M1244 t470 t469 vdd vdd pch w=2u l=180n
CT473 t473 0 0.1f
M1245 t470 nw76 t473 0 nch w=1u l=180n
M1246 t473 t469 0 0 nch w=1u l=180n
M1247 t471 nw94 vdd vdd pch w=2u l=180n
M1248 t471 t469 vdd vdd pch w=2u l=180n
CT474 t474 0 0.1f
M1249 t471 nw94 t474 0 nch w=1u l=180n
M1250 t474 t469 0 0 nch w=1u l=180n
M1251 nw152 t470 vdd vdd pch w=2u l=180n
M1252 nw152 t471 vdd vdd pch w=2u l=180n
CT475 t475 0 0.1f
M1253 nw152 t470 t475 0 nch w=1u l=180n
M1254 t475 t471 0 0 nch w=1u l=180n
Cnw152 nw152 0 2f
M1255 nw153 nw78 vdd vdd pch w=2u l=180n
M1256 nw153 nw97 vdd vdd pch w=2u l=180n
CT476 t476 0 0.1f
M1257 nw153 nw78 t476 0 nch w=1u l=180n
M1258 t476 nw97 0 0 nch w=1u l=180n
Cnw153 nw153 0 2f
M1259 nw154 nw80 0 0 nch w=1u l=180n
M1260 nw154 nw100 0 0 nch w=1u l=180n
CT477 t477 0 0.1f
M1261 t477 nw80 vdd vdd pch w=2u l=180n
M1262 nw154 nw100 t477 vdd pch w=2u l=180n
Cnw154 nw154 0 2f
CT478 t478 0 0.1f
M1263 t478 nw82 vdd vdd pch w=2u l=180n
M1264 t478 nw103 vdd vdd pch w=2u l=180n
CT479 t479 0 0.1f
M1265 t478 nw82 t479 0 nch w=1u l=180n
M1266 t479 nw103 0 0 nch w=1u l=180n
M1267 nw155 t478 vdd vdd pch w=2u l=180n
M1268 nw155 t478 0 0 nch w=1u l=180n
Cnw155 nw155 0 2f
CT480 t480 0 0.1f
M1269 t480 nw84 0 0 nch w=1u l=180n
M1270 t480 nw106 0 0 nch w=1u l=180n
CT481 t481 0 0.1f
M1271 t481 nw84 vdd vdd pch w=2u l=180n
M1272 t480 nw106 t481 vdd pch w=2u l=180n
M1273 nw156 t480 vdd vdd pch w=2u l=180n
M1274 nw156 t480 0 0 nch w=1u l=180n
Cnw156 nw156 0 2f
CT482 t482 0 0.1f
CT483 t483 0 0.1f
CT484 t484 0 0.1f
M1275 t482 nw86 vdd vdd pch w=2u l=180n
M1276 t482 nw109 vdd vdd pch w=2u l=180n
CT485 t485 0 0.1f
M1277 t482 nw86 t485 0 nch w=1u l=180n
M1278 t485 nw109 0 0 nch w=1u l=180n
M1279 t483 nw86 vdd vdd pch w=2u l=180n
M1280 t483 t482 vdd vdd pch w=2u l=180n
CT486 t486 0 0.1f
M1281 t483 nw86 t486 0 nch w=1u l=180n
M1282 t486 t482 0 0 nch w=1u l=180n
M1283 t484 nw109 vdd vdd pch w=2u l=180n
M1284 t484 t482 vdd vdd pch w=2u l=180n
CT487 t487 0 0.1f
M1285 t484 nw109 t487 0 nch w=1u l=180n
M1286 t487 t482 0 0 nch w=1u l=180n
M1287 nw157 t483 vdd vdd pch w=2u l=180n
M1288 nw157 t484 vdd vdd pch w=2u l=180n
CT488 t488 0 0.1f
M1289 nw157 t483 t488 0 nch w=1u l=180n
M1290 t488 t484 0 0 nch w=1u l=180n
Cnw157 nw157 0 2f
M1291 nw158 nw88 vdd vdd pch w=2u l=180n
M1292 nw158 nw112 vdd vdd pch w=2u l=180n
CT489 t489 0 0.1f
M1293 nw158 nw88 t489 0 nch w=1u l=180n
M1294 t489 nw112 0 0 nch w=1u l=180n
Cnw158 nw158 0 2f
M1295 nw159 nw90 0 0 nch w=1u l=180n
M1296 nw159 nw115 0 0 nch w=1u l=180n
CT490 t490 0 0.1f
M1297 t490 nw90 vdd vdd pch w=2u l=180n
M1298 nw159 nw115 t490 vdd pch w=2u l=180n
Cnw159 nw159 0 2f
CT491 t491 0 0.1f
M1299 t491 nw92 vdd vdd pch w=2u l=180n
M1300 t491 nw118 vdd vdd pch w=2u l=180n
CT492 t492 0 0.1f
M1301 t491 nw92 t492 0 nch w=1u l=180n
M1302 t492 nw118 0 0 nch w=1u l=180n
M1303 nw160 t491 vdd vdd pch w=2u l=180n
M1304 nw160 t491 0 0 nch w=1u l=180n
Cnw160 nw160 0 2f
CT493 t493 0 0.1f
M1305 t493 nw94 0 0 nch w=1u l=180n
M1306 t493 nw121 0 0 nch w=1u l=180n
CT494 t494 0 0.1f
M1307 t494 nw94 vdd vdd pch w=2u l=180n
M1308 t493 nw121 t494 vdd pch w=2u l=180n
M1309 nw161 t493 vdd vdd pch w=2u l=180n
M1310 nw161 t493 0 0 nch w=1u l=180n
Cnw161 nw161 0 2f
CT495 t495 0 0.1f
CT496 t496 0 0.1f
CT497 t497 0 0.1f
M1311 t495 nw96 vdd vdd pch w=2u l=180n
M1312 t495 nw124 vdd vdd pch w=2u l=180n
CT498 t498 0 0.1f
M1313 t495 nw96 t498 0 nch w=1u l=180n
M1314 t498 nw124 0 0 nch w=1u l=180n
M1315 t496 nw96 vdd vdd pch w=2u l=180n
M1316 t496 t495 vdd vdd pch w=2u l=180n
CT499 t499 0 0.1f
M1317 t496 nw96 t499 0 nch w=1u l=180n
M1318 t499 t495 0 0 nch w=1u l=180n
M1319 t497 nw124 vdd vdd pch w=2u l=180n
M1320 t497 t495 vdd vdd pch w=2u l=180n
CT500 t500 0 0.1f
M1321 t497 nw124 t500 0 nch w=1u l=180n
M1322 t500 t495 0 0 nch w=1u l=180n
M1323 nw162 t496 vdd vdd pch w=2u l=180n
M1324 nw162 t497 vdd vdd pch w=2u l=180n
CT501 t501 0 0.1f
M1325 nw162 t496 t501 0 nch w=1u l=180n
M1326 t501 t497 0 0 nch w=1u l=180n
Cnw162 nw162 0 2f
M1327 nw163 nw98 vdd vdd pch w=2u l=180n
M1328 nw163 nw127 vdd vdd pch w=2u l=180n
CT502 t502 0 0.1f
M1329 nw163 nw98 t502 0 nch w=1u l=180n
M1330 t502 nw127 0 0 nch w=1u l=180n
Cnw163 nw163 0 2f
M1331 nw164 nw100 0 0 nch w=1u l=180n
M1332 nw164 nw130 0 0 nch w=1u l=180n
CT503 t503 0 0.1f
M1333 t503 nw100 vdd vdd pch w=2u l=180n
M1334 nw164 nw130 t503 vdd pch w=2u l=180n
Cnw164 nw164 0 2f
CT504 t504 0 0.1f
M1335 t504 nw102 vdd vdd pch w=2u l=180n
M1336 t504 nw133 vdd vdd pch w=2u l=180n
CT505 t505 0 0.1f
M1337 t504 nw102 t505 0 nch w=1u l=180n
M1338 t505 nw133 0 0 nch w=1u l=180n
M1339 nw165 t504 vdd vdd pch w=2u l=180n
M1340 nw165 t504 0 0 nch w=1u l=180n
Cnw165 nw165 0 2f
CT506 t506 0 0.1f
M1341 t506 nw104 0 0 nch w=1u l=180n
M1342 t506 nw136 0 0 nch w=1u l=180n
CT507 t507 0 0.1f
M1343 t507 nw104 vdd vdd pch w=2u l=180n
M1344 t506 nw136 t507 vdd pch w=2u l=180n
M1345 nw166 t506 vdd vdd pch w=2u l=180n
M1346 nw166 t506 0 0 nch w=1u l=180n
Cnw166 nw166 0 2f
CT508 t508 0 0.1f
CT509 t509 0 0.1f
CT510 t510 0 0.1f
M1347 t508 nw106 vdd vdd pch w=2u l=180n
M1348 t508 nw139 vdd vdd pch w=2u l=180n
CT511 t511 0 0.1f
M1349 t508 nw106 t511 0 nch w=1u l=180n
M1350 t511 nw139 0 0 nch w=1u l=180n
M1351 t509 nw106 vdd vdd pch w=2u l=180n
M1352 t509 t508 vdd vdd pch w=2u l=180n
CT512 t512 0 0.1f
M1353 t509 nw106 t512 0 nch w=1u l=180n
M1354 t512 t508 0 0 nch w=1u l=180n
M1355 t510 nw139 vdd vdd pch w=2u l=180n
M1356 t510 t508 vdd vdd pch w=2u l=180n
CT513 t513 0 0.1f
M1357 t510 nw139 t513 0 nch w=1u l=180n
M1358 t513 t508 0 0 nch w=1u l=180n
M1359 nw167 t509 vdd vdd pch w=2u l=180n
M1360 nw167 t510 vdd vdd pch w=2u l=180n
CT514 t514 0 0.1f
M1361 nw167 t509 t514 0 nch w=1u l=180n
M1362 t514 t510 0 0 nch w=1u l=180n
Cnw167 nw167 0 2f
M1363 nw168 nw108 vdd vdd pch w=2u l=180n
M1364 nw168 nw142 vdd vdd pch w=2u l=180n
CT515 t515 0 0.1f
M1365 nw168 nw108 t515 0 nch w=1u l=180n
M1366 t515 nw142 0 0 nch w=1u l=180n
Cnw168 nw168 0 2f
M1367 nw169 nw110 0 0 nch w=1u l=180n
M1368 nw169 nw145 0 0 nch w=1u l=180n
CT516 t516 0 0.1f
M1369 t516 nw110 vdd vdd pch w=2u l=180n
M1370 nw169 nw145 t516 vdd pch w=2u l=180n
Cnw169 nw169 0 2f
CT517 t517 0 0.1f
M1371 t517 nw112 vdd vdd pch w=2u l=180n
M1372 t517 nw148 vdd vdd pch w=2u l=180n
CT518 t518 0 0.1f
M1373 t517 nw112 t518 0 nch w=1u l=180n
M1374 t518 nw148 0 0 nch w=1u l=180n
M1375 nw170 t517 vdd vdd pch w=2u l=180n
M1376 nw170 t517 0 0 nch w=1u l=180n
Cnw170 nw170 0 2f
CT519 t519 0 0.1f
M1377 t519 nw114 0 0 nch w=1u l=180n
M1378 t519 nw151 0 0 nch w=1u l=180n
CT520 t520 0 0.1f
M1379 t520 nw114 vdd vdd pch w=2u l=180n
M1380 t519 nw151 t520 vdd pch w=2u l=180n
M1381 nw171 t519 vdd vdd pch w=2u l=180n
M1382 nw171 t519 0 0 nch w=1u l=180n
Cnw171 nw171 0 2f
CT521 t521 0 0.1f
CT522 t522 0 0.1f
CT523 t523 0 0.1f
M1383 t521 nw116 vdd vdd pch w=2u l=180n
M1384 t521 nw154 vdd vdd pch w=2u l=180n
CT524 t524 0 0.1f
M1385 t521 nw116 t524 0 nch w=1u l=180n
M1386 t524 nw154 0 0 nch w=1u l=180n
M1387 t522 nw116 vdd vdd pch w=2u l=180n
M1388 t522 t521 vdd vdd pch w=2u l=180n
CT525 t525 0 0.1f
M1389 t522 nw116 t525 0 nch w=1u l=180n
M1390 t525 t521 0 0 nch w=1u l=180n
M1391 t523 nw154 vdd vdd pch w=2u l=180n
M1392 t523 t521 vdd vdd pch w=2u l=180n
CT526 t526 0 0.1f
M1393 t523 nw154 t526 0 nch w=1u l=180n
M1394 t526 t521 0 0 nch w=1u l=180n
M1395 nw172 t522 vdd vdd pch w=2u l=180n
M1396 nw172 t523 vdd vdd pch w=2u l=180n
CT527 t527 0 0.1f
M1397 nw172 t522 t527 0 nch w=1u l=180n
M1398 t527 t523 0 0 nch w=1u l=180n
Cnw172 nw172 0 2f
M1399 nw173 nw118 vdd vdd pch w=2u l=180n
M1400 nw173 nw157 vdd vdd pch w=2u l=180n
CT528 t528 0 0.1f
M1401 nw173 nw118 t528 0 nch w=1u l=180n
M1402 t528 nw157 0 0 nch w=1u l=180n
Cnw173 nw173 0 2f
M1403 nw174 nw120 0 0 nch w=1u l=180n
M1404 nw174 nw160 0 0 nch w=1u l=180n
CT529 t529 0 0.1f
M1405 t529 nw120 vdd vdd pch w=2u l=180n
M1406 nw174 nw160 t529 vdd pch w=2u l=180n
Cnw174 nw174 0 2f
CT530 t530 0 0.1f
M1407 t530 nw122 vdd vdd pch w=2u l=180n
M1408 t530 nw163 vdd vdd pch w=2u l=180n
CT531 t531 0 0.1f
M1409 t530 nw122 t531 0 nch w=1u l=180n
M1410 t531 nw163 0 0 nch w=1u l=180n
M1411 nw175 t530 vdd vdd pch w=2u l=180n
M1412 nw175 t530 0 0 nch w=1u l=180n
Cnw175 nw175 0 2f
CT532 t532 0 0.1f
M1413 t532 nw124 0 0 nch w=1u l=180n
M1414 t532 nw166 0 0 nch w=1u l=180n
CT533 t533 0 0.1f
M1415 t533 nw124 vdd vdd pch w=2u l=180n
M1416 t532 nw166 t533 vdd pch w=2u l=180n
M1417 nw176 t532 vdd vdd pch w=2u l=180n
M1418 nw176 t532 0 0 nch w=1u l=180n
Cnw176 nw176 0 2f
CT534 t534 0 0.1f
CT535 t535 0 0.1f
CT536 t536 0 0.1f
M1419 t534 nw126 vdd vdd pch w=2u l=180n
M1420 t534 nw169 vdd vdd pch w=2u l=180n
CT537 t537 0 0.1f
M1421 t534 nw126 t537 0 nch w=1u l=180n
M1422 t537 nw169 0 0 nch w=1u l=180n
M1423 t535 nw126 vdd vdd pch w=2u l=180n
M1424 t535 t534 vdd vdd pch w=2u l=180n
CT538 t538 0 0.1f
M1425 t535 nw126 t538 0 nch w=1u l=180n
M1426 t538 t534 0 0 nch w=1u l=180n
M1427 t536 nw169 vdd vdd pch w=2u l=180n
M1428 t536 t534 vdd vdd pch w=2u l=180n
CT539 t539 0 0.1f
M1429 t536 nw169 t539 0 nch w=1u l=180n
M1430 t539 t534 0 0 nch w=1u l=180n
M1431 nw177 t535 vdd vdd pch w=2u l=180n
M1432 nw177 t536 vdd vdd pch w=2u l=180n
CT540 t540 0 0.1f
M1433 nw177 t535 t540 0 nch w=1u l=180n
M1434 t540 t536 0 0 nch w=1u l=180n
Cnw177 nw177 0 2f
M1435 nw178 nw128 vdd vdd pch w=2u l=180n
M1436 nw178 nw172 vdd vdd pch w=2u l=180n
CT541 t541 0 0.1f
M1437 nw178 nw128 t541 0 nch w=1u l=180n
M1438 t541 nw172 0 0 nch w=1u l=180n
Cnw178 nw178 0 2f
M1439 nw179 nw130 0 0 nch w=1u l=180n
M1440 nw179 nw175 0 0 nch w=1u l=180n
CT542 t542 0 0.1f
M1441 t542 nw130 vdd vdd pch w=2u l=180n
M1442 nw179 nw175 t542 vdd pch w=2u l=180n
Cnw179 nw179 0 2f
CT543 t543 0 0.1f
M1443 t543 nw132 vdd vdd pch w=2u l=180n
M1444 t543 nw178 vdd vdd pch w=2u l=180n
CT544 t544 0 0.1f
M1445 t543 nw132 t544 0 nch w=1u l=180n
M1446 t544 nw178 0 0 nch w=1u l=180n
M1447 nw180 t543 vdd vdd pch w=2u l=180n
M1448 nw180 t543 0 0 nch w=1u l=180n
Cnw180 nw180 0 2f
CT545 t545 0 0.1f
M1449 t545 nw134 0 0 nch w=1u l=180n
M1450 t545 nq0 0 0 nch w=1u l=180n
CT546 t546 0 0.1f
M1451 t546 nw134 vdd vdd pch w=2u l=180n
M1452 t545 nq0 t546 vdd pch w=2u l=180n
M1453 nw181 t545 vdd vdd pch w=2u l=180n
M1454 nw181 t545 0 0 nch w=1u l=180n
Cnw181 nw181 0 2f
CT547 t547 0 0.1f
CT548 t548 0 0.1f
CT549 t549 0 0.1f
M1455 t547 nw136 vdd vdd pch w=2u l=180n
M1456 t547 nq2 vdd vdd pch w=2u l=180n
CT550 t550 0 0.1f
M1457 t547 nw136 t550 0 nch w=1u l=180n
M1458 t550 nq2 0 0 nch w=1u l=180n
M1459 t548 nw136 vdd vdd pch w=2u l=180n
M1460 t548 t547 vdd vdd pch w=2u l=180n
CT551 t551 0 0.1f
M1461 t548 nw136 t551 0 nch w=1u l=180n
M1462 t551 t547 0 0 nch w=1u l=180n
M1463 t549 nq2 vdd vdd pch w=2u l=180n
M1464 t549 t547 vdd vdd pch w=2u l=180n
CT552 t552 0 0.1f
M1465 t549 nq2 t552 0 nch w=1u l=180n
M1466 t552 t547 0 0 nch w=1u l=180n
M1467 nw182 t548 vdd vdd pch w=2u l=180n
M1468 nw182 t549 vdd vdd pch w=2u l=180n
CT553 t553 0 0.1f
M1469 nw182 t548 t553 0 nch w=1u l=180n
M1470 t553 t549 0 0 nch w=1u l=180n
Cnw182 nw182 0 2f
CT554 t554 0 0.1f
M1471 t554 nw182 vdd vdd pch w=2u l=180n
M1472 t554 nw182 0 0 nch w=1u l=180n
M1473 no0 t554 vdd vdd pch w=2u l=180n
M1474 no0 t554 0 0 nch w=1u l=180n
Cno0 no0 0 2f
CT555 t555 0 0.1f
M1475 t555 nw181 vdd vdd pch w=2u l=180n
M1476 t555 nw181 0 0 nch w=1u l=180n
M1477 no1 t555 vdd vdd pch w=2u l=180n
M1478 no1 t555 0 0 nch w=1u l=180n
Cno1 no1 0 2f
CT556 t556 0 0.1f
M1479 t556 nw180 vdd vdd pch w=2u l=180n
M1480 t556 nw180 0 0 nch w=1u l=180n
M1481 no2 t556 vdd vdd pch w=2u l=180n
M1482 no2 t556 0 0 nch w=1u l=180n
Cno2 no2 0 2f
CT557 t557 0 0.1f
M1483 t557 nw179 vdd vdd pch w=2u l=180n
M1484 t557 nw179 0 0 nch w=1u l=180n
M1485 no3 t557 vdd vdd pch w=2u l=180n
M1486 no3 t557 0 0 nch w=1u l=180n
Cno3 no3 0 2f
CT558 t558 0 0.1f
M1487 t558 nw178 vdd vdd pch w=2u l=180n
M1488 t558 nw178 0 0 nch w=1u l=180n
M1489 no4 t558 vdd vdd pch w=2u l=180n
M1490 no4 t558 0 0 nch w=1u l=180n
Cno4 no4 0 2f
CT559 t559 0 0.1f
M1491 t559 nw177 vdd vdd pch w=2u l=180n
M1492 t559 nw177 0 0 nch w=1u l=180n
M1493 no5 t559 vdd vdd pch w=2u l=180n
M1494 no5 t559 0 0 nch w=1u l=180n
Cno5 no5 0 2f
CT560 t560 0 0.1f
M1495 t560 nw176 vdd vdd pch w=2u l=180n
M1496 t560 nw176 0 0 nch w=1u l=180n
M1497 no6 t560 vdd vdd pch w=2u l=180n
M1498 no6 t560 0 0 nch w=1u l=180n
Cno6 no6 0 2f
CT561 t561 0 0.1f
M1499 t561 nw175 vdd vdd pch w=2u l=180n
M1500 t561 nw175 0 0 nch w=1u l=180n
M1501 no7 t561 vdd vdd pch w=2u l=180n
M1502 no7 t561 0 0 nch w=1u l=180n
Cno7 no7 0 2f
.model nch NMOS (vto=0.45 kp=200u lambda=0.05)
.model pch PMOS (vto=-0.45 kp=100u lambda=0.05)
* outputs: nw1 nw3 nw5 nw7 nw9 nw11 nw13 nw15 nw17 nw19 nw21 nw23 nw25 nw27 nw29 nw31 nw33 nw35 nw37 nw39 nw41 no0 no1 no2 no3 no4 no5 no6 no7
.end
