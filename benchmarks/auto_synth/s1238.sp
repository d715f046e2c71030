* s1238 (s1238: 18 flip-flops, 508 gates): 510 gates, 3664 transistors
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
VIN9 nq0 0 PULSE(0 1.8 2.56e-07 20p 20p 5.12e-07 1.024e-06)
VIN10 nq1 0 PULSE(0 1.8 5.12e-07 20p 20p 1.024e-06 2.048e-06)
VIN11 nq2 0 PULSE(0 1.8 1.024e-06 20p 20p 2.048e-06 4.096e-06)
VIN12 nq3 0 PULSE(0 1.8 2.048e-06 20p 20p 4.096e-06 8.192e-06)
VIN13 nq4 0 PULSE(0 1.8 4.096e-06 20p 20p 8.192e-06 1.6384e-05)
VIN14 nq5 0 PULSE(0 1.8 8.192e-06 20p 20p 1.6384e-05 3.2768e-05)
VIN15 nq6 0 PULSE(0 1.8 1.6384e-05 20p 20p 3.2768e-05 6.5536e-05)
VIN16 nq7 0 PULSE(0 1.8 3.2768e-05 20p 20p 6.5536e-05 0.000131072)
VIN17 nq8 0 PULSE(0 1.8 6.5536e-05 20p 20p 0.000131072 0.000262144)
VIN18 nq9 0 PULSE(0 1.8 0.000131072 20p 20p 0.000262144 0.000524288)
VIN19 nq10 0 PULSE(0 1.8 0.000262144 20p 20p 0.000524288 0.001048576)
VIN20 nq11 0 PULSE(0 1.8 0.000524288 20p 20p 0.001048576 0.002097152)
VIN21 nq12 0 PULSE(0 1.8 0.001048576 20p 20p 0.002097152 0.004194304)
VIN22 nq13 0 PULSE(0 1.8 0.002097152 20p 20p 0.004194304 0.008388608)
VIN23 nq14 0 PULSE(0 1.8 0.004194304 20p 20p 0.008388608 0.016777216)
VIN24 nq15 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN25 nq16 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN26 nq17 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
CT1 t1 0 0.1f
CT2 t2 0 0.1f
CT3 t3 0 0.1f
M1 t1 nq17 vdd vdd pch w=2u l=180n
M2 t1 nq9 vdd vdd pch w=2u l=180n
CT4 t4 0 0.1f
M3 t1 nq17 t4 0 nch w=1u l=180n
M4 t4 nq9 0 0 nch w=1u l=180n
M5 t2 nq17 vdd vdd pch w=2u l=180n
M6 t2 t1 vdd vdd pch w=2u l=180n
CT5 t5 0 0.1f
M7 t2 nq17 t5 0 nch w=1u l=180n
M8 t5 t1 0 0 nch w=1u l=180n
M9 t3 nq9 vdd vdd pch w=2u l=180n
M10 t3 t1 vdd vdd pch w=2u l=180n
CT6 t6 0 0.1f
M11 t3 nq9 t6 0 nch w=1u l=180n
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
M18 t8 ni0 vdd vdd pch w=2u l=180n
CT11 t11 0 0.1f
M19 t8 nw1 t11 0 nch w=1u l=180n
M20 t11 ni0 0 0 nch w=1u l=180n
M21 t9 nw1 vdd vdd pch w=2u l=180n
M22 t9 t8 vdd vdd pch w=2u l=180n
CT12 t12 0 0.1f
M23 t9 nw1 t12 0 nch w=1u l=180n
M24 t12 t8 0 0 nch w=1u l=180n
M25 t10 ni0 vdd vdd pch w=2u l=180n
M26 t10 t8 vdd vdd pch w=2u l=180n
CT13 t13 0 0.1f
M27 t10 ni0 t13 0 nch w=1u l=180n
M28 t13 t8 0 0 nch w=1u l=180n
M29 nw2 t9 vdd vdd pch w=2u l=180n
M30 nw2 t10 vdd vdd pch w=2u l=180n
CT14 t14 0 0.1f
M31 nw2 t9 t14 0 nch w=1u l=180n
M32 t14 t10 0 0 nch w=1u l=180n
Cnw2 nw2 0 2f
M33 nw3 nq1 vdd vdd pch w=2u l=180n
M34 nw3 nq3 vdd vdd pch w=2u l=180n
CT15 t15 0 0.1f
M35 nw3 nq1 t15 0 nch w=1u l=180n
M36 t15 nq3 0 0 nch w=1u l=180n
Cnw3 nw3 0 2f
M37 nw4 nq8 0 0 nch w=1u l=180n
M38 nw4 nq14 0 0 nch w=1u l=180n
CT16 t16 0 0.1f
M39 t16 nq8 vdd vdd pch w=2u l=180n
M40 nw4 nq14 t16 vdd pch w=2u l=180n
Cnw4 nw4 0 2f
CT17 t17 0 0.1f
M41 t17 nq15 vdd vdd pch w=2u l=180n
M42 t17 ni7 vdd vdd pch w=2u l=180n
CT18 t18 0 0.1f
M43 t17 nq15 t18 0 nch w=1u l=180n
M44 t18 ni7 0 0 nch w=1u l=180n
M45 nw5 t17 vdd vdd pch w=2u l=180n
M46 nw5 t17 0 0 nch w=1u l=180n
Cnw5 nw5 0 2f
CT19 t19 0 0.1f
M47 t19 ni4 0 0 nch w=1u l=180n
M48 t19 nq6 0 0 nch w=1u l=180n
CT20 t20 0 0.1f
M49 t20 ni4 vdd vdd pch w=2u l=180n
M50 t19 nq6 t20 vdd pch w=2u l=180n
M51 nw6 t19 vdd vdd pch w=2u l=180n
M52 nw6 t19 0 0 nch w=1u l=180n
Cnw6 nw6 0 2f
CT21 t21 0 0.1f
CT22 t22 0 0.1f
CT23 t23 0 0.1f
M53 t21 nw5 vdd vdd pch w=2u l=180n
M54 t21 nq16 vdd vdd pch w=2u l=180n
CT24 t24 0 0.1f
M55 t21 nw5 t24 0 nch w=1u l=180n
M56 t24 nq16 0 0 nch w=1u l=180n
M57 t22 nw5 vdd vdd pch w=2u l=180n
M58 t22 t21 vdd vdd pch w=2u l=180n
CT25 t25 0 0.1f
M59 t22 nw5 t25 0 nch w=1u l=180n
M60 t25 t21 0 0 nch w=1u l=180n
M61 t23 nq16 vdd vdd pch w=2u l=180n
M62 t23 t21 vdd vdd pch w=2u l=180n
CT26 t26 0 0.1f
M63 t23 nq16 t26 0 nch w=1u l=180n
M64 t26 t21 0 0 nch w=1u l=180n
M65 nw7 t22 vdd vdd pch w=2u l=180n
M66 nw7 t23 vdd vdd pch w=2u l=180n
CT27 t27 0 0.1f
M67 nw7 t22 t27 0 nch w=1u l=180n
M68 t27 t23 0 0 nch w=1u l=180n
Cnw7 nw7 0 2f
M69 nw8 nq4 vdd vdd pch w=2u l=180n
M70 nw8 ni8 vdd vdd pch w=2u l=180n
CT28 t28 0 0.1f
M71 nw8 nq4 t28 0 nch w=1u l=180n
M72 t28 ni8 0 0 nch w=1u l=180n
Cnw8 nw8 0 2f
M73 nw9 nq10 0 0 nch w=1u l=180n
M74 nw9 nq3 0 0 nch w=1u l=180n
CT29 t29 0 0.1f
M75 t29 nq10 vdd vdd pch w=2u l=180n
M76 nw9 nq3 t29 vdd pch w=2u l=180n
Cnw9 nw9 0 2f
CT30 t30 0 0.1f
M77 t30 nq16 vdd vdd pch w=2u l=180n
M78 t30 nq12 vdd vdd pch w=2u l=180n
CT31 t31 0 0.1f
M79 t30 nq16 t31 0 nch w=1u l=180n
M80 t31 nq12 0 0 nch w=1u l=180n
M81 nw10 t30 vdd vdd pch w=2u l=180n
M82 nw10 t30 0 0 nch w=1u l=180n
Cnw10 nw10 0 2f
CT32 t32 0 0.1f
M83 t32 ni4 0 0 nch w=1u l=180n
M84 t32 ni3 0 0 nch w=1u l=180n
CT33 t33 0 0.1f
M85 t33 ni4 vdd vdd pch w=2u l=180n
M86 t32 ni3 t33 vdd pch w=2u l=180n
M87 nw11 t32 vdd vdd pch w=2u l=180n
M88 nw11 t32 0 0 nch w=1u l=180n
Cnw11 nw11 0 2f
CT34 t34 0 0.1f
CT35 t35 0 0.1f
CT36 t36 0 0.1f
M89 t34 nw4 vdd vdd pch w=2u l=180n
M90 t34 nw6 vdd vdd pch w=2u l=180n
CT37 t37 0 0.1f
M91 t34 nw4 t37 0 nch w=1u l=180n
M92 t37 nw6 0 0 nch w=1u l=180n
M93 t35 nw4 vdd vdd pch w=2u l=180n
M94 t35 t34 vdd vdd pch w=2u l=180n
CT38 t38 0 0.1f
M95 t35 nw4 t38 0 nch w=1u l=180n
M96 t38 t34 0 0 nch w=1u l=180n
M97 t36 nw6 vdd vdd pch w=2u l=180n
M98 t36 t34 vdd vdd pch w=2u l=180n
CT39 t39 0 0.1f
M99 t36 nw6 t39 0 nch w=1u l=180n
M100 t39 t34 0 0 nch w=1u l=180n
M101 nw12 t35 vdd vdd pch w=2u l=180n
M102 nw12 t36 vdd vdd pch w=2u l=180n
CT40 t40 0 0.1f
M103 nw12 t35 t40 0 nch w=1u l=180n
M104 t40 t36 0 0 nch w=1u l=180n
Cnw12 nw12 0 2f
M105 nw13 nw10 vdd vdd pch w=2u l=180n
M106 nw13 nq2 vdd vdd pch w=2u l=180n
CT41 t41 0 0.1f
M107 nw13 nw10 t41 0 nch w=1u l=180n
M108 t41 nq2 0 0 nch w=1u l=180n
Cnw13 nw13 0 2f
M109 nw14 nq2 0 0 nch w=1u l=180n
M110 nw14 nq10 0 0 nch w=1u l=180n
CT42 t42 0 0.1f
M111 t42 nq2 vdd vdd pch w=2u l=180n
M112 nw14 nq10 t42 vdd pch w=2u l=180n
Cnw14 nw14 0 2f
CT43 t43 0 0.1f
M113 t43 nq7 vdd vdd pch w=2u l=180n
M114 t43 ni0 vdd vdd pch w=2u l=180n
CT44 t44 0 0.1f
M115 t43 nq7 t44 0 nch w=1u l=180n
M116 t44 ni0 0 0 nch w=1u l=180n
M117 nw15 t43 vdd vdd pch w=2u l=180n
M118 nw15 t43 0 0 nch w=1u l=180n
Cnw15 nw15 0 2f
CT45 t45 0 0.1f
M119 t45 nq12 0 0 nch w=1u l=180n
M120 t45 ni8 0 0 nch w=1u l=180n
CT46 t46 0 0.1f
M121 t46 nq12 vdd vdd pch w=2u l=180n
M122 t45 ni8 t46 vdd pch w=2u l=180n
M123 nw16 t45 vdd vdd pch w=2u l=180n
M124 nw16 t45 0 0 nch w=1u l=180n
Cnw16 nw16 0 2f
CT47 t47 0 0.1f
CT48 t48 0 0.1f
CT49 t49 0 0.1f
M125 t47 nq17 vdd vdd pch w=2u l=180n
M126 t47 nw10 vdd vdd pch w=2u l=180n
CT50 t50 0 0.1f
M127 t47 nq17 t50 0 nch w=1u l=180n
M128 t50 nw10 0 0 nch w=1u l=180n
M129 t48 nq17 vdd vdd pch w=2u l=180n
M130 t48 t47 vdd vdd pch w=2u l=180n
CT51 t51 0 0.1f
M131 t48 nq17 t51 0 nch w=1u l=180n
M132 t51 t47 0 0 nch w=1u l=180n
M133 t49 nw10 vdd vdd pch w=2u l=180n
M134 t49 t47 vdd vdd pch w=2u l=180n
CT52 t52 0 0.1f
M135 t49 nw10 t52 0 nch w=1u l=180n
M136 t52 t47 0 0 nch w=1u l=180n
M137 nw17 t48 vdd vdd pch w=2u l=180n
M138 nw17 t49 vdd vdd pch w=2u l=180n
CT53 t53 0 0.1f
M139 nw17 t48 t53 0 nch w=1u l=180n
M140 t53 t49 0 0 nch w=1u l=180n
Cnw17 nw17 0 2f
M141 nw18 ni4 vdd vdd pch w=2u l=180n
M142 nw18 nq0 vdd vdd pch w=2u l=180n
CT54 t54 0 0.1f
M143 nw18 ni4 t54 0 nch w=1u l=180n
M144 t54 nq0 0 0 nch w=1u l=180n
Cnw18 nw18 0 2f
M145 nw19 nw3 0 0 nch w=1u l=180n
M146 nw19 nq7 0 0 nch w=1u l=180n
CT55 t55 0 0.1f
M147 t55 nw3 vdd vdd pch w=2u l=180n
M148 nw19 nq7 t55 vdd pch w=2u l=180n
Cnw19 nw19 0 2f
CT56 t56 0 0.1f
M149 t56 nw8 vdd vdd pch w=2u l=180n
M150 t56 nq14 vdd vdd pch w=2u l=180n
CT57 t57 0 0.1f
M151 t56 nw8 t57 0 nch w=1u l=180n
M152 t57 nq14 0 0 nch w=1u l=180n
M153 nw20 t56 vdd vdd pch w=2u l=180n
M154 nw20 t56 0 0 nch w=1u l=180n
Cnw20 nw20 0 2f
CT58 t58 0 0.1f
M155 t58 nw13 0 0 nch w=1u l=180n
M156 t58 ni3 0 0 nch w=1u l=180n
CT59 t59 0 0.1f
M157 t59 nw13 vdd vdd pch w=2u l=180n
M158 t58 ni3 t59 vdd pch w=2u l=180n
M159 nw21 t58 vdd vdd pch w=2u l=180n
M160 nw21 t58 0 0 nch w=1u l=180n
Cnw21 nw21 0 2f
CT60 t60 0 0.1f
CT61 t61 0 0.1f
CT62 t62 0 0.1f
M161 t60 nw18 vdd vdd pch w=2u l=180n
M162 t60 nw4 vdd vdd pch w=2u l=180n
CT63 t63 0 0.1f
M163 t60 nw18 t63 0 nch w=1u l=180n
M164 t63 nw4 0 0 nch w=1u l=180n
M165 t61 nw18 vdd vdd pch w=2u l=180n
M166 t61 t60 vdd vdd pch w=2u l=180n
CT64 t64 0 0.1f
M167 t61 nw18 t64 0 nch w=1u l=180n
M168 t64 t60 0 0 nch w=1u l=180n
M169 t62 nw4 vdd vdd pch w=2u l=180n
M170 t62 t60 vdd vdd pch w=2u l=180n
CT65 t65 0 0.1f
M171 t62 nw4 t65 0 nch w=1u l=180n
M172 t65 t60 0 0 nch w=1u l=180n
M173 nw22 t61 vdd vdd pch w=2u l=180n
M174 nw22 t62 vdd vdd pch w=2u l=180n
CT66 t66 0 0.1f
M175 nw22 t61 t66 0 nch w=1u l=180n
M176 t66 t62 0 0 nch w=1u l=180n
Cnw22 nw22 0 2f
M177 nw23 nq0 vdd vdd pch w=2u l=180n
M178 nw23 nw11 vdd vdd pch w=2u l=180n
CT67 t67 0 0.1f
M179 nw23 nq0 t67 0 nch w=1u l=180n
M180 t67 nw11 0 0 nch w=1u l=180n
Cnw23 nw23 0 2f
M181 nw24 nq4 0 0 nch w=1u l=180n
M182 nw24 nw18 0 0 nch w=1u l=180n
CT68 t68 0 0.1f
M183 t68 nq4 vdd vdd pch w=2u l=180n
M184 nw24 nw18 t68 vdd pch w=2u l=180n
Cnw24 nw24 0 2f
CT69 t69 0 0.1f
M185 t69 nq8 vdd vdd pch w=2u l=180n
M186 t69 nq0 vdd vdd pch w=2u l=180n
CT70 t70 0 0.1f
M187 t69 nq8 t70 0 nch w=1u l=180n
M188 t70 nq0 0 0 nch w=1u l=180n
M189 nw25 t69 vdd vdd pch w=2u l=180n
M190 nw25 t69 0 0 nch w=1u l=180n
Cnw25 nw25 0 2f
CT71 t71 0 0.1f
M191 t71 nq12 0 0 nch w=1u l=180n
M192 t71 nq6 0 0 nch w=1u l=180n
CT72 t72 0 0.1f
M193 t72 nq12 vdd vdd pch w=2u l=180n
M194 t71 nq6 t72 vdd pch w=2u l=180n
M195 nw26 t71 vdd vdd pch w=2u l=180n
M196 nw26 t71 0 0 nch w=1u l=180n
Cnw26 nw26 0 2f
CT73 t73 0 0.1f
CT74 t74 0 0.1f
CT75 t75 0 0.1f
M197 t73 nq16 vdd vdd pch w=2u l=180n
M198 t73 nq12 vdd vdd pch w=2u l=180n
CT76 t76 0 0.1f
M199 t73 nq16 t76 0 nch w=1u l=180n
M200 t76 nq12 0 0 nch w=1u l=180n
M201 t74 nq16 vdd vdd pch w=2u l=180n
M202 t74 t73 vdd vdd pch w=2u l=180n
CT77 t77 0 0.1f
M203 t74 nq16 t77 0 nch w=1u l=180n
M204 t77 t73 0 0 nch w=1u l=180n
M205 t75 nq12 vdd vdd pch w=2u l=180n
M206 t75 t73 vdd vdd pch w=2u l=180n
CT78 t78 0 0.1f
M207 t75 nq12 t78 0 nch w=1u l=180n
M208 t78 t73 0 0 nch w=1u l=180n
M209 nw27 t74 vdd vdd pch w=2u l=180n
M210 nw27 t75 vdd vdd pch w=2u l=180n
CT79 t79 0 0.1f
M211 nw27 t74 t79 0 nch w=1u l=180n
M212 t79 t75 0 0 nch w=1u l=180n
Cnw27 nw27 0 2f
M213 nw28 ni2 vdd vdd pch w=2u l=180n
M214 nw28 ni0 vdd vdd pch w=2u l=180n
CT80 t80 0 0.1f
M215 nw28 ni2 t80 0 nch w=1u l=180n
M216 t80 ni0 0 0 nch w=1u l=180n
Cnw28 nw28 0 2f
M217 nw29 ni6 0 0 nch w=1u l=180n
M218 nw29 ni7 0 0 nch w=1u l=180n
CT81 t81 0 0.1f
M219 t81 ni6 vdd vdd pch w=2u l=180n
M220 nw29 ni7 t81 vdd pch w=2u l=180n
Cnw29 nw29 0 2f
CT82 t82 0 0.1f
M221 t82 nw4 vdd vdd pch w=2u l=180n
M222 t82 nw6 vdd vdd pch w=2u l=180n
CT83 t83 0 0.1f
M223 t82 nw4 t83 0 nch w=1u l=180n
M224 t83 nw6 0 0 nch w=1u l=180n
M225 nw30 t82 vdd vdd pch w=2u l=180n
M226 nw30 t82 0 0 nch w=1u l=180n
Cnw30 nw30 0 2f
CT84 t84 0 0.1f
M227 t84 nw8 0 0 nch w=1u l=180n
M228 t84 nw12 0 0 nch w=1u l=180n
CT85 t85 0 0.1f
M229 t85 nw8 vdd vdd pch w=2u l=180n
M230 t84 nw12 t85 vdd pch w=2u l=180n
M231 nw31 t84 vdd vdd pch w=2u l=180n
M232 nw31 t84 0 0 nch w=1u l=180n
Cnw31 nw31 0 2f
CT86 t86 0 0.1f
CT87 t87 0 0.1f
CT88 t88 0 0.1f
M233 t86 nw12 vdd vdd pch w=2u l=180n
M234 t86 nw18 vdd vdd pch w=2u l=180n
CT89 t89 0 0.1f
M235 t86 nw12 t89 0 nch w=1u l=180n
M236 t89 nw18 0 0 nch w=1u l=180n
M237 t87 nw12 vdd vdd pch w=2u l=180n
M238 t87 t86 vdd vdd pch w=2u l=180n
CT90 t90 0 0.1f
M239 t87 nw12 t90 0 nch w=1u l=180n
M240 t90 t86 0 0 nch w=1u l=180n
M241 t88 nw18 vdd vdd pch w=2u l=180n
M242 t88 t86 vdd vdd pch w=2u l=180n
CT91 t91 0 0.1f
M243 t88 nw18 t91 0 nch w=1u l=180n
M244 t91 t86 0 0 nch w=1u l=180n
M245 nw32 t87 vdd vdd pch w=2u l=180n
M246 nw32 t88 vdd vdd pch w=2u l=180n
CT92 t92 0 0.1f
M247 nw32 t87 t92 0 nch w=1u l=180n
M248 t92 t88 0 0 nch w=1u l=180n
Cnw32 nw32 0 2f
M249 nw33 nw16 vdd vdd pch w=2u l=180n
M250 nw33 nw24 vdd vdd pch w=2u l=180n
CT93 t93 0 0.1f
M251 nw33 nw16 t93 0 nch w=1u l=180n
M252 t93 nw24 0 0 nch w=1u l=180n
Cnw33 nw33 0 2f
M253 nw34 nw20 0 0 nch w=1u l=180n
M254 nw34 nw30 0 0 nch w=1u l=180n
CT94 t94 0 0.1f
M255 t94 nw20 vdd vdd pch w=2u l=180n
M256 nw34 nw30 t94 vdd pch w=2u l=180n
Cnw34 nw34 0 2f
CT95 t95 0 0.1f
M257 t95 nw24 vdd vdd pch w=2u l=180n
M258 t95 nq1 vdd vdd pch w=2u l=180n
CT96 t96 0 0.1f
M259 t95 nw24 t96 0 nch w=1u l=180n
M260 t96 nq1 0 0 nch w=1u l=180n
M261 nw35 t95 vdd vdd pch w=2u l=180n
M262 nw35 t95 0 0 nch w=1u l=180n
Cnw35 nw35 0 2f
CT97 t97 0 0.1f
M263 t97 nw28 0 0 nch w=1u l=180n
M264 t97 nq6 0 0 nch w=1u l=180n
CT98 t98 0 0.1f
M265 t98 nw28 vdd vdd pch w=2u l=180n
M266 t97 nq6 t98 vdd pch w=2u l=180n
M267 nw36 t97 vdd vdd pch w=2u l=180n
M268 nw36 t97 0 0 nch w=1u l=180n
Cnw36 nw36 0 2f
CT99 t99 0 0.1f
CT100 t100 0 0.1f
CT101 t101 0 0.1f
M269 t99 nw32 vdd vdd pch w=2u l=180n
M270 t99 nq11 vdd vdd pch w=2u l=180n
CT102 t102 0 0.1f
M271 t99 nw32 t102 0 nch w=1u l=180n
M272 t102 nq11 0 0 nch w=1u l=180n
M273 t100 nw32 vdd vdd pch w=2u l=180n
M274 t100 t99 vdd vdd pch w=2u l=180n
CT103 t103 0 0.1f
M275 t100 nw32 t103 0 nch w=1u l=180n
M276 t103 t99 0 0 nch w=1u l=180n
M277 t101 nq11 vdd vdd pch w=2u l=180n
M278 t101 t99 vdd vdd pch w=2u l=180n
CT104 t104 0 0.1f
M279 t101 nq11 t104 0 nch w=1u l=180n
M280 t104 t99 0 0 nch w=1u l=180n
M281 nw37 t100 vdd vdd pch w=2u l=180n
M282 nw37 t101 vdd vdd pch w=2u l=180n
CT105 t105 0 0.1f
M283 nw37 t100 t105 0 nch w=1u l=180n
M284 t105 t101 0 0 nch w=1u l=180n
Cnw37 nw37 0 2f
M285 nw38 nw36 vdd vdd pch w=2u l=180n
M286 nw38 nq16 vdd vdd pch w=2u l=180n
CT106 t106 0 0.1f
M287 nw38 nw36 t106 0 nch w=1u l=180n
M288 t106 nq16 0 0 nch w=1u l=180n
Cnw38 nw38 0 2f
M289 nw39 nq1 0 0 nch w=1u l=180n
M290 nw39 ni3 0 0 nch w=1u l=180n
CT107 t107 0 0.1f
M291 t107 nq1 vdd vdd pch w=2u l=180n
M292 nw39 ni3 t107 vdd pch w=2u l=180n
Cnw39 nw39 0 2f
CT108 t108 0 0.1f
M293 t108 nq4 vdd vdd pch w=2u l=180n
M294 t108 ni8 vdd vdd pch w=2u l=180n
CT109 t109 0 0.1f
M295 t108 nq4 t109 0 nch w=1u l=180n
M296 t109 ni8 0 0 nch w=1u l=180n
M297 nw40 t108 vdd vdd pch w=2u l=180n
M298 nw40 t108 0 0 nch w=1u l=180n
Cnw40 nw40 0 2f
CT110 t110 0 0.1f
M299 t110 nq7 0 0 nch w=1u l=180n
M300 t110 nw7 0 0 nch w=1u l=180n
CT111 t111 0 0.1f
M301 t111 nq7 vdd vdd pch w=2u l=180n
M302 t110 nw7 t111 vdd pch w=2u l=180n
M303 nw41 t110 vdd vdd pch w=2u l=180n
M304 nw41 t110 0 0 nch w=1u l=180n
Cnw41 nw41 0 2f
CT112 t112 0 0.1f
CT113 t113 0 0.1f
CT114 t114 0 0.1f
M305 t112 nq10 vdd vdd pch w=2u l=180n
M306 t112 nw12 vdd vdd pch w=2u l=180n
CT115 t115 0 0.1f
M307 t112 nq10 t115 0 nch w=1u l=180n
M308 t115 nw12 0 0 nch w=1u l=180n
M309 t113 nq10 vdd vdd pch w=2u l=180n
M310 t113 t112 vdd vdd pch w=2u l=180n
CT116 t116 0 0.1f
M311 t113 nq10 t116 0 nch w=1u l=180n
M312 t116 t112 0 0 nch w=1u l=180n
M313 t114 nw12 vdd vdd pch w=2u l=180n
M314 t114 t112 vdd vdd pch w=2u l=180n
CT117 t117 0 0.1f
M315 t114 nw12 t117 0 nch w=1u l=180n
M316 t117 t112 0 0 nch w=1u l=180n
M317 nw42 t113 vdd vdd pch w=2u l=180n
M318 nw42 t114 vdd vdd pch w=2u l=180n
CT118 t118 0 0.1f
M319 nw42 t113 t118 0 nch w=1u l=180n
M320 t118 t114 0 0 nch w=1u l=180n
Cnw42 nw42 0 2f
M321 nw43 nq13 vdd vdd pch w=2u l=180n
M322 nw43 nw17 vdd vdd pch w=2u l=180n
CT119 t119 0 0.1f
M323 nw43 nq13 t119 0 nch w=1u l=180n
M324 t119 nw17 0 0 nch w=1u l=180n
Cnw43 nw43 0 2f
M325 nw44 nq16 0 0 nch w=1u l=180n
M326 nw44 nw22 0 0 nch w=1u l=180n
CT120 t120 0 0.1f
M327 t120 nq16 vdd vdd pch w=2u l=180n
M328 nw44 nw22 t120 vdd pch w=2u l=180n
Cnw44 nw44 0 2f
CT121 t121 0 0.1f
M329 t121 ni1 vdd vdd pch w=2u l=180n
M330 t121 nw27 vdd vdd pch w=2u l=180n
CT122 t122 0 0.1f
M331 t121 ni1 t122 0 nch w=1u l=180n
M332 t122 nw27 0 0 nch w=1u l=180n
M333 nw45 t121 vdd vdd pch w=2u l=180n
M334 nw45 t121 0 0 nch w=1u l=180n
Cnw45 nw45 0 2f
CT123 t123 0 0.1f
M335 t123 ni4 0 0 nch w=1u l=180n
M336 t123 nw32 0 0 nch w=1u l=180n
CT124 t124 0 0.1f
M337 t124 ni4 vdd vdd pch w=2u l=180n
M338 t123 nw32 t124 vdd pch w=2u l=180n
M339 nw46 t123 vdd vdd pch w=2u l=180n
M340 nw46 t123 0 0 nch w=1u l=180n
Cnw46 nw46 0 2f
CT125 t125 0 0.1f
CT126 t126 0 0.1f
CT127 t127 0 0.1f
M341 t125 ni7 vdd vdd pch w=2u l=180n
M342 t125 nw37 vdd vdd pch w=2u l=180n
CT128 t128 0 0.1f
M343 t125 ni7 t128 0 nch w=1u l=180n
M344 t128 nw37 0 0 nch w=1u l=180n
M345 t126 ni7 vdd vdd pch w=2u l=180n
M346 t126 t125 vdd vdd pch w=2u l=180n
CT129 t129 0 0.1f
M347 t126 ni7 t129 0 nch w=1u l=180n
M348 t129 t125 0 0 nch w=1u l=180n
M349 t127 nw37 vdd vdd pch w=2u l=180n
M350 t127 t125 vdd vdd pch w=2u l=180n
CT130 t130 0 0.1f
M351 t127 nw37 t130 0 nch w=1u l=180n
M352 t130 t125 0 0 nch w=1u l=180n
M353 nw47 t126 vdd vdd pch w=2u l=180n
M354 nw47 t127 vdd vdd pch w=2u l=180n
CT131 t131 0 0.1f
M355 nw47 t126 t131 0 nch w=1u l=180n
M356 t131 t127 0 0 nch w=1u l=180n
Cnw47 nw47 0 2f
M357 nw48 nw4 vdd vdd pch w=2u l=180n
M358 nw48 nw42 vdd vdd pch w=2u l=180n
CT132 t132 0 0.1f
M359 nw48 nw4 t132 0 nch w=1u l=180n
M360 t132 nw42 0 0 nch w=1u l=180n
Cnw48 nw48 0 2f
M361 nw49 nw7 0 0 nch w=1u l=180n
M362 nw49 nw47 0 0 nch w=1u l=180n
CT133 t133 0 0.1f
M363 t133 nw7 vdd vdd pch w=2u l=180n
M364 nw49 nw47 t133 vdd pch w=2u l=180n
Cnw49 nw49 0 2f
CT134 t134 0 0.1f
M365 t134 nw10 vdd vdd pch w=2u l=180n
M366 t134 nq2 vdd vdd pch w=2u l=180n
CT135 t135 0 0.1f
M367 t134 nw10 t135 0 nch w=1u l=180n
M368 t135 nq2 0 0 nch w=1u l=180n
M369 nw50 t134 vdd vdd pch w=2u l=180n
M370 nw50 t134 0 0 nch w=1u l=180n
Cnw50 nw50 0 2f
CT136 t136 0 0.1f
M371 t136 nw13 0 0 nch w=1u l=180n
M372 t136 nq6 0 0 nch w=1u l=180n
CT137 t137 0 0.1f
M373 t137 nw13 vdd vdd pch w=2u l=180n
M374 t136 nq6 t137 vdd pch w=2u l=180n
M375 nw51 t136 vdd vdd pch w=2u l=180n
M376 nw51 t136 0 0 nch w=1u l=180n
Cnw51 nw51 0 2f
CT138 t138 0 0.1f
CT139 t139 0 0.1f
CT140 t140 0 0.1f
M377 t138 nw16 vdd vdd pch w=2u l=180n
M378 t138 nq10 vdd vdd pch w=2u l=180n
CT141 t141 0 0.1f
M379 t138 nw16 t141 0 nch w=1u l=180n
M380 t141 nq10 0 0 nch w=1u l=180n
M381 t139 nw16 vdd vdd pch w=2u l=180n
M382 t139 t138 vdd vdd pch w=2u l=180n
CT142 t142 0 0.1f
M383 t139 nw16 t142 0 nch w=1u l=180n
M384 t142 t138 0 0 nch w=1u l=180n
M385 t140 nq10 vdd vdd pch w=2u l=180n
M386 t140 t138 vdd vdd pch w=2u l=180n
CT143 t143 0 0.1f
M387 t140 nq10 t143 0 nch w=1u l=180n
M388 t143 t138 0 0 nch w=1u l=180n
M389 nw52 t139 vdd vdd pch w=2u l=180n
M390 nw52 t140 vdd vdd pch w=2u l=180n
CT144 t144 0 0.1f
M391 nw52 t139 t144 0 nch w=1u l=180n
M392 t144 t140 0 0 nch w=1u l=180n
Cnw52 nw52 0 2f
M393 nw53 nw19 vdd vdd pch w=2u l=180n
M394 nw53 nq14 vdd vdd pch w=2u l=180n
CT145 t145 0 0.1f
M395 nw53 nw19 t145 0 nch w=1u l=180n
M396 t145 nq14 0 0 nch w=1u l=180n
Cnw53 nw53 0 2f
M397 nw54 nw22 0 0 nch w=1u l=180n
M398 nw54 ni0 0 0 nch w=1u l=180n
CT146 t146 0 0.1f
M399 t146 nw22 vdd vdd pch w=2u l=180n
M400 nw54 ni0 t146 vdd pch w=2u l=180n
Cnw54 nw54 0 2f
CT147 t147 0 0.1f
M401 t147 nw25 vdd vdd pch w=2u l=180n
M402 t147 ni4 vdd vdd pch w=2u l=180n
CT148 t148 0 0.1f
M403 t147 nw25 t148 0 nch w=1u l=180n
M404 t148 ni4 0 0 nch w=1u l=180n
M405 nw55 t147 vdd vdd pch w=2u l=180n
M406 nw55 t147 0 0 nch w=1u l=180n
Cnw55 nw55 0 2f
CT149 t149 0 0.1f
M407 t149 nw28 0 0 nch w=1u l=180n
M408 t149 ni8 0 0 nch w=1u l=180n
CT150 t150 0 0.1f
M409 t150 nw28 vdd vdd pch w=2u l=180n
M410 t149 ni8 t150 vdd pch w=2u l=180n
M411 nw56 t149 vdd vdd pch w=2u l=180n
M412 nw56 t149 0 0 nch w=1u l=180n
Cnw56 nw56 0 2f
CT151 t151 0 0.1f
CT152 t152 0 0.1f
CT153 t153 0 0.1f
M413 t151 nw31 vdd vdd pch w=2u l=180n
M414 t151 nw6 vdd vdd pch w=2u l=180n
CT154 t154 0 0.1f
M415 t151 nw31 t154 0 nch w=1u l=180n
M416 t154 nw6 0 0 nch w=1u l=180n
M417 t152 nw31 vdd vdd pch w=2u l=180n
M418 t152 t151 vdd vdd pch w=2u l=180n
CT155 t155 0 0.1f
M419 t152 nw31 t155 0 nch w=1u l=180n
M420 t155 t151 0 0 nch w=1u l=180n
M421 t153 nw6 vdd vdd pch w=2u l=180n
M422 t153 t151 vdd vdd pch w=2u l=180n
CT156 t156 0 0.1f
M423 t153 nw6 t156 0 nch w=1u l=180n
M424 t156 t151 0 0 nch w=1u l=180n
M425 nw57 t152 vdd vdd pch w=2u l=180n
M426 nw57 t153 vdd vdd pch w=2u l=180n
CT157 t157 0 0.1f
M427 nw57 t152 t157 0 nch w=1u l=180n
M428 t157 t153 0 0 nch w=1u l=180n
Cnw57 nw57 0 2f
M429 nw58 nw34 vdd vdd pch w=2u l=180n
M430 nw58 nw10 vdd vdd pch w=2u l=180n
CT158 t158 0 0.1f
M431 nw58 nw34 t158 0 nch w=1u l=180n
M432 t158 nw10 0 0 nch w=1u l=180n
Cnw58 nw58 0 2f
M433 nw59 nw37 0 0 nch w=1u l=180n
M434 nw59 nw14 0 0 nch w=1u l=180n
CT159 t159 0 0.1f
M435 t159 nw37 vdd vdd pch w=2u l=180n
M436 nw59 nw14 t159 vdd pch w=2u l=180n
Cnw59 nw59 0 2f
CT160 t160 0 0.1f
M437 t160 nw40 vdd vdd pch w=2u l=180n
M438 t160 nw18 vdd vdd pch w=2u l=180n
CT161 t161 0 0.1f
M439 t160 nw40 t161 0 nch w=1u l=180n
M440 t161 nw18 0 0 nch w=1u l=180n
M441 nw60 t160 vdd vdd pch w=2u l=180n
M442 nw60 t160 0 0 nch w=1u l=180n
Cnw60 nw60 0 2f
CT162 t162 0 0.1f
M443 t162 nw43 0 0 nch w=1u l=180n
M444 t162 nw22 0 0 nch w=1u l=180n
CT163 t163 0 0.1f
M445 t163 nw43 vdd vdd pch w=2u l=180n
M446 t162 nw22 t163 vdd pch w=2u l=180n
M447 nw61 t162 vdd vdd pch w=2u l=180n
M448 nw61 t162 0 0 nch w=1u l=180n
Cnw61 nw61 0 2f
CT164 t164 0 0.1f
CT165 t165 0 0.1f
CT166 t166 0 0.1f
M449 t164 nw46 vdd vdd pch w=2u l=180n
M450 t164 nw26 vdd vdd pch w=2u l=180n
CT167 t167 0 0.1f
M451 t164 nw46 t167 0 nch w=1u l=180n
M452 t167 nw26 0 0 nch w=1u l=180n
M453 t165 nw46 vdd vdd pch w=2u l=180n
M454 t165 t164 vdd vdd pch w=2u l=180n
CT168 t168 0 0.1f
M455 t165 nw46 t168 0 nch w=1u l=180n
M456 t168 t164 0 0 nch w=1u l=180n
M457 t166 nw26 vdd vdd pch w=2u l=180n
M458 t166 t164 vdd vdd pch w=2u l=180n
CT169 t169 0 0.1f
M459 t166 nw26 t169 0 nch w=1u l=180n
M460 t169 t164 0 0 nch w=1u l=180n
M461 nw62 t165 vdd vdd pch w=2u l=180n
M462 nw62 t166 vdd vdd pch w=2u l=180n
CT170 t170 0 0.1f
M463 nw62 t165 t170 0 nch w=1u l=180n
M464 t170 t166 0 0 nch w=1u l=180n
Cnw62 nw62 0 2f
M465 nw63 nw49 vdd vdd pch w=2u l=180n
M466 nw63 nw30 vdd vdd pch w=2u l=180n
CT171 t171 0 0.1f
M467 nw63 nw49 t171 0 nch w=1u l=180n
M468 t171 nw30 0 0 nch w=1u l=180n
Cnw63 nw63 0 2f
M469 nw64 nw52 0 0 nch w=1u l=180n
M470 nw64 nw34 0 0 nch w=1u l=180n
CT172 t172 0 0.1f
M471 t172 nw52 vdd vdd pch w=2u l=180n
M472 nw64 nw34 t172 vdd pch w=2u l=180n
Cnw64 nw64 0 2f
CT173 t173 0 0.1f
M473 t173 nw55 vdd vdd pch w=2u l=180n
M474 t173 nw38 vdd vdd pch w=2u l=180n
CT174 t174 0 0.1f
M475 t173 nw55 t174 0 nch w=1u l=180n
M476 t174 nw38 0 0 nch w=1u l=180n
M477 nw65 t173 vdd vdd pch w=2u l=180n
M478 nw65 t173 0 0 nch w=1u l=180n
Cnw65 nw65 0 2f
CT175 t175 0 0.1f
M479 t175 nw58 0 0 nch w=1u l=180n
M480 t175 nw42 0 0 nch w=1u l=180n
CT176 t176 0 0.1f
M481 t176 nw58 vdd vdd pch w=2u l=180n
M482 t175 nw42 t176 vdd pch w=2u l=180n
M483 nw66 t175 vdd vdd pch w=2u l=180n
M484 nw66 t175 0 0 nch w=1u l=180n
Cnw66 nw66 0 2f
CT177 t177 0 0.1f
CT178 t178 0 0.1f
CT179 t179 0 0.1f
M485 t177 nw61 vdd vdd pch w=2u l=180n
M486 t177 nw46 vdd vdd pch w=2u l=180n
CT180 t180 0 0.1f
M487 t177 nw61 t180 0 nch w=1u l=180n
M488 t180 nw46 0 0 nch w=1u l=180n
M489 t178 nw61 vdd vdd pch w=2u l=180n
M490 t178 t177 vdd vdd pch w=2u l=180n
CT181 t181 0 0.1f
M491 t178 nw61 t181 0 nch w=1u l=180n
M492 t181 t177 0 0 nch w=1u l=180n
M493 t179 nw46 vdd vdd pch w=2u l=180n
M494 t179 t177 vdd vdd pch w=2u l=180n
CT182 t182 0 0.1f
M495 t179 nw46 t182 0 nch w=1u l=180n
M496 t182 t177 0 0 nch w=1u l=180n
M497 nw67 t178 vdd vdd pch w=2u l=180n
M498 nw67 t179 vdd vdd pch w=2u l=180n
CT183 t183 0 0.1f
M499 nw67 t178 t183 0 nch w=1u l=180n
M500 t183 t179 0 0 nch w=1u l=180n
Cnw67 nw67 0 2f
M501 nw68 nw64 vdd vdd pch w=2u l=180n
M502 nw68 nw50 vdd vdd pch w=2u l=180n
CT184 t184 0 0.1f
M503 nw68 nw64 t184 0 nch w=1u l=180n
M504 t184 nw50 0 0 nch w=1u l=180n
Cnw68 nw68 0 2f
M505 nw69 nw67 0 0 nch w=1u l=180n
M506 nw69 nw54 0 0 nch w=1u l=180n
CT185 t185 0 0.1f
M507 t185 nw67 vdd vdd pch w=2u l=180n
M508 nw69 nw54 t185 vdd pch w=2u l=180n
Cnw69 nw69 0 2f
CT186 t186 0 0.1f
M509 t186 nq0 vdd vdd pch w=2u l=180n
M510 t186 nw58 vdd vdd pch w=2u l=180n
CT187 t187 0 0.1f
M511 t186 nq0 t187 0 nch w=1u l=180n
M512 t187 nw58 0 0 nch w=1u l=180n
M513 nw70 t186 vdd vdd pch w=2u l=180n
M514 nw70 t186 0 0 nch w=1u l=180n
Cnw70 nw70 0 2f
CT188 t188 0 0.1f
M515 t188 nq2 0 0 nch w=1u l=180n
M516 t188 nw62 0 0 nch w=1u l=180n
CT189 t189 0 0.1f
M517 t189 nq2 vdd vdd pch w=2u l=180n
M518 t188 nw62 t189 vdd pch w=2u l=180n
M519 nw71 t188 vdd vdd pch w=2u l=180n
M520 nw71 t188 0 0 nch w=1u l=180n
Cnw71 nw71 0 2f
CT190 t190 0 0.1f
CT191 t191 0 0.1f
CT192 t192 0 0.1f
M521 t190 nq4 vdd vdd pch w=2u l=180n
M522 t190 nw66 vdd vdd pch w=2u l=180n
CT193 t193 0 0.1f
M523 t190 nq4 t193 0 nch w=1u l=180n
M524 t193 nw66 0 0 nch w=1u l=180n
M525 t191 nq4 vdd vdd pch w=2u l=180n
M526 t191 t190 vdd vdd pch w=2u l=180n
CT194 t194 0 0.1f
M527 t191 nq4 t194 0 nch w=1u l=180n
M528 t194 t190 0 0 nch w=1u l=180n
M529 t192 nw66 vdd vdd pch w=2u l=180n
M530 t192 t190 vdd vdd pch w=2u l=180n
CT195 t195 0 0.1f
M531 t192 nw66 t195 0 nch w=1u l=180n
M532 t195 t190 0 0 nch w=1u l=180n
M533 nw72 t191 vdd vdd pch w=2u l=180n
M534 nw72 t192 vdd vdd pch w=2u l=180n
CT196 t196 0 0.1f
M535 nw72 t191 t196 0 nch w=1u l=180n
M536 t196 t192 0 0 nch w=1u l=180n
Cnw72 nw72 0 2f
M537 nw73 nq6 vdd vdd pch w=2u l=180n
M538 nw73 nw70 vdd vdd pch w=2u l=180n
CT197 t197 0 0.1f
M539 nw73 nq6 t197 0 nch w=1u l=180n
M540 t197 nw70 0 0 nch w=1u l=180n
Cnw73 nw73 0 2f
M541 nw74 nq8 0 0 nch w=1u l=180n
M542 nw74 nq0 0 0 nch w=1u l=180n
CT198 t198 0 0.1f
M543 t198 nq8 vdd vdd pch w=2u l=180n
M544 nw74 nq0 t198 vdd pch w=2u l=180n
Cnw74 nw74 0 2f
CT199 t199 0 0.1f
M545 t199 nq10 vdd vdd pch w=2u l=180n
M546 t199 nq3 vdd vdd pch w=2u l=180n
CT200 t200 0 0.1f
M547 t199 nq10 t200 0 nch w=1u l=180n
M548 t200 nq3 0 0 nch w=1u l=180n
M549 nw75 t199 vdd vdd pch w=2u l=180n
M550 nw75 t199 0 0 nch w=1u l=180n
Cnw75 nw75 0 2f
CT201 t201 0 0.1f
M551 t201 nq12 0 0 nch w=1u l=180n
M552 t201 nq6 0 0 nch w=1u l=180n
CT202 t202 0 0.1f
M553 t202 nq12 vdd vdd pch w=2u l=180n
M554 t201 nq6 t202 vdd pch w=2u l=180n
M555 nw76 t201 vdd vdd pch w=2u l=180n
M556 nw76 t201 0 0 nch w=1u l=180n
Cnw76 nw76 0 2f
CT203 t203 0 0.1f
CT204 t204 0 0.1f
CT205 t205 0 0.1f
M557 t203 nq14 vdd vdd pch w=2u l=180n
M558 t203 nq9 vdd vdd pch w=2u l=180n
CT206 t206 0 0.1f
M559 t203 nq14 t206 0 nch w=1u l=180n
M560 t206 nq9 0 0 nch w=1u l=180n
M561 t204 nq14 vdd vdd pch w=2u l=180n
M562 t204 t203 vdd vdd pch w=2u l=180n
CT207 t207 0 0.1f
M563 t204 nq14 t207 0 nch w=1u l=180n
M564 t207 t203 0 0 nch w=1u l=180n
M565 t205 nq9 vdd vdd pch w=2u l=180n
M566 t205 t203 vdd vdd pch w=2u l=180n
CT208 t208 0 0.1f
M567 t205 nq9 t208 0 nch w=1u l=180n
M568 t208 t203 0 0 nch w=1u l=180n
M569 nw77 t204 vdd vdd pch w=2u l=180n
M570 nw77 t205 vdd vdd pch w=2u l=180n
CT209 t209 0 0.1f
M571 nw77 t204 t209 0 nch w=1u l=180n
M572 t209 t205 0 0 nch w=1u l=180n
Cnw77 nw77 0 2f
M573 nw78 nq16 vdd vdd pch w=2u l=180n
M574 nw78 nq12 vdd vdd pch w=2u l=180n
CT210 t210 0 0.1f
M575 nw78 nq16 t210 0 nch w=1u l=180n
M576 t210 nq12 0 0 nch w=1u l=180n
Cnw78 nw78 0 2f
M577 nw79 ni0 0 0 nch w=1u l=180n
M578 nw79 nq15 0 0 nch w=1u l=180n
CT211 t211 0 0.1f
M579 t211 ni0 vdd vdd pch w=2u l=180n
M580 nw79 nq15 t211 vdd pch w=2u l=180n
Cnw79 nw79 0 2f
CT212 t212 0 0.1f
M581 t212 ni2 vdd vdd pch w=2u l=180n
M582 t212 ni0 vdd vdd pch w=2u l=180n
CT213 t213 0 0.1f
M583 t212 ni2 t213 0 nch w=1u l=180n
M584 t213 ni0 0 0 nch w=1u l=180n
M585 nw80 t212 vdd vdd pch w=2u l=180n
M586 nw80 t212 0 0 nch w=1u l=180n
Cnw80 nw80 0 2f
CT214 t214 0 0.1f
M587 t214 ni4 0 0 nch w=1u l=180n
M588 t214 ni3 0 0 nch w=1u l=180n
CT215 t215 0 0.1f
M589 t215 ni4 vdd vdd pch w=2u l=180n
M590 t214 ni3 t215 vdd pch w=2u l=180n
M591 nw81 t214 vdd vdd pch w=2u l=180n
M592 nw81 t214 0 0 nch w=1u l=180n
Cnw81 nw81 0 2f
CT216 t216 0 0.1f
CT217 t217 0 0.1f
CT218 t218 0 0.1f
M593 t216 ni6 vdd vdd pch w=2u l=180n
M594 t216 nw54 vdd vdd pch w=2u l=180n
CT219 t219 0 0.1f
M595 t216 ni6 t219 0 nch w=1u l=180n
M596 t219 nw54 0 0 nch w=1u l=180n
M597 t217 ni6 vdd vdd pch w=2u l=180n
M598 t217 t216 vdd vdd pch w=2u l=180n
CT220 t220 0 0.1f
M599 t217 ni6 t220 0 nch w=1u l=180n
M600 t220 t216 0 0 nch w=1u l=180n
M601 t218 nw54 vdd vdd pch w=2u l=180n
M602 t218 t216 vdd vdd pch w=2u l=180n
CT221 t221 0 0.1f
M603 t218 nw54 t221 0 nch w=1u l=180n
M604 t221 t216 0 0 nch w=1u l=180n
M605 nw82 t217 vdd vdd pch w=2u l=180n
M606 nw82 t218 vdd vdd pch w=2u l=180n
CT222 t222 0 0.1f
M607 nw82 t217 t222 0 nch w=1u l=180n
M608 t222 t218 0 0 nch w=1u l=180n
Cnw82 nw82 0 2f
M609 nw83 ni8 vdd vdd pch w=2u l=180n
M610 nw83 nw3 vdd vdd pch w=2u l=180n
CT223 t223 0 0.1f
M611 nw83 ni8 t223 0 nch w=1u l=180n
M612 t223 nw3 0 0 nch w=1u l=180n
Cnw83 nw83 0 2f
M613 nw84 nw4 0 0 nch w=1u l=180n
M614 nw84 nw6 0 0 nch w=1u l=180n
CT224 t224 0 0.1f
M615 t224 nw4 vdd vdd pch w=2u l=180n
M616 nw84 nw6 t224 vdd pch w=2u l=180n
Cnw84 nw84 0 2f
CT225 t225 0 0.1f
M617 t225 nw6 vdd vdd pch w=2u l=180n
M618 t225 nw9 vdd vdd pch w=2u l=180n
CT226 t226 0 0.1f
M619 t225 nw6 t226 0 nch w=1u l=180n
M620 t226 nw9 0 0 nch w=1u l=180n
M621 nw85 t225 vdd vdd pch w=2u l=180n
M622 nw85 t225 0 0 nch w=1u l=180n
Cnw85 nw85 0 2f
CT227 t227 0 0.1f
M623 t227 nw8 0 0 nch w=1u l=180n
M624 t227 nw12 0 0 nch w=1u l=180n
CT228 t228 0 0.1f
M625 t228 nw8 vdd vdd pch w=2u l=180n
M626 t227 nw12 t228 vdd pch w=2u l=180n
M627 nw86 t227 vdd vdd pch w=2u l=180n
M628 nw86 t227 0 0 nch w=1u l=180n
Cnw86 nw86 0 2f
CT229 t229 0 0.1f
CT230 t230 0 0.1f
CT231 t231 0 0.1f
M629 t229 nw10 vdd vdd pch w=2u l=180n
M630 t229 nw15 vdd vdd pch w=2u l=180n
CT232 t232 0 0.1f
M631 t229 nw10 t232 0 nch w=1u l=180n
M632 t232 nw15 0 0 nch w=1u l=180n
M633 t230 nw10 vdd vdd pch w=2u l=180n
M634 t230 t229 vdd vdd pch w=2u l=180n
CT233 t233 0 0.1f
M635 t230 nw10 t233 0 nch w=1u l=180n
M636 t233 t229 0 0 nch w=1u l=180n
M637 t231 nw15 vdd vdd pch w=2u l=180n
M638 t231 t229 vdd vdd pch w=2u l=180n
CT234 t234 0 0.1f
M639 t231 nw15 t234 0 nch w=1u l=180n
M640 t234 t229 0 0 nch w=1u l=180n
M641 nw87 t230 vdd vdd pch w=2u l=180n
M642 nw87 t231 vdd vdd pch w=2u l=180n
CT235 t235 0 0.1f
M643 nw87 t230 t235 0 nch w=1u l=180n
M644 t235 t231 0 0 nch w=1u l=180n
Cnw87 nw87 0 2f
M645 nw88 nw12 vdd vdd pch w=2u l=180n
M646 nw88 nw18 vdd vdd pch w=2u l=180n
CT236 t236 0 0.1f
M647 nw88 nw12 t236 0 nch w=1u l=180n
M648 t236 nw18 0 0 nch w=1u l=180n
Cnw88 nw88 0 2f
M649 nw89 nw14 0 0 nch w=1u l=180n
M650 nw89 nw21 0 0 nch w=1u l=180n
CT237 t237 0 0.1f
M651 t237 nw14 vdd vdd pch w=2u l=180n
M652 nw89 nw21 t237 vdd pch w=2u l=180n
Cnw89 nw89 0 2f
CT238 t238 0 0.1f
M653 t238 nw16 vdd vdd pch w=2u l=180n
M654 t238 nw24 vdd vdd pch w=2u l=180n
CT239 t239 0 0.1f
M655 t238 nw16 t239 0 nch w=1u l=180n
M656 t239 nw24 0 0 nch w=1u l=180n
M657 nw90 t238 vdd vdd pch w=2u l=180n
M658 nw90 t238 0 0 nch w=1u l=180n
Cnw90 nw90 0 2f
CT240 t240 0 0.1f
M659 t240 nw18 0 0 nch w=1u l=180n
M660 t240 nw27 0 0 nch w=1u l=180n
CT241 t241 0 0.1f
M661 t241 nw18 vdd vdd pch w=2u l=180n
M662 t240 nw27 t241 vdd pch w=2u l=180n
M663 nw91 t240 vdd vdd pch w=2u l=180n
M664 nw91 t240 0 0 nch w=1u l=180n
Cnw91 nw91 0 2f
CT242 t242 0 0.1f
CT243 t243 0 0.1f
CT244 t244 0 0.1f
M665 t242 nw20 vdd vdd pch w=2u l=180n
M666 t242 nw30 vdd vdd pch w=2u l=180n
CT245 t245 0 0.1f
M667 t242 nw20 t245 0 nch w=1u l=180n
M668 t245 nw30 0 0 nch w=1u l=180n
M669 t243 nw20 vdd vdd pch w=2u l=180n
M670 t243 t242 vdd vdd pch w=2u l=180n
CT246 t246 0 0.1f
M671 t243 nw20 t246 0 nch w=1u l=180n
M672 t246 t242 0 0 nch w=1u l=180n
M673 t244 nw30 vdd vdd pch w=2u l=180n
M674 t244 t242 vdd vdd pch w=2u l=180n
CT247 t247 0 0.1f
M675 t244 nw30 t247 0 nch w=1u l=180n
M676 t247 t242 0 0 nch w=1u l=180n
M677 nw92 t243 vdd vdd pch w=2u l=180n
M678 nw92 t244 vdd vdd pch w=2u l=180n
CT248 t248 0 0.1f
M679 nw92 t243 t248 0 nch w=1u l=180n
M680 t248 t244 0 0 nch w=1u l=180n
Cnw92 nw92 0 2f
M681 nw93 nw22 vdd vdd pch w=2u l=180n
M682 nw93 nw33 vdd vdd pch w=2u l=180n
CT249 t249 0 0.1f
M683 nw93 nw22 t249 0 nch w=1u l=180n
M684 t249 nw33 0 0 nch w=1u l=180n
Cnw93 nw93 0 2f
M685 nw94 nw24 0 0 nch w=1u l=180n
M686 nw94 nw36 0 0 nch w=1u l=180n
CT250 t250 0 0.1f
M687 t250 nw24 vdd vdd pch w=2u l=180n
M688 nw94 nw36 t250 vdd pch w=2u l=180n
Cnw94 nw94 0 2f
CT251 t251 0 0.1f
M689 t251 nw26 vdd vdd pch w=2u l=180n
M690 t251 nw39 vdd vdd pch w=2u l=180n
CT252 t252 0 0.1f
M691 t251 nw26 t252 0 nch w=1u l=180n
M692 t252 nw39 0 0 nch w=1u l=180n
M693 nw95 t251 vdd vdd pch w=2u l=180n
M694 nw95 t251 0 0 nch w=1u l=180n
Cnw95 nw95 0 2f
CT253 t253 0 0.1f
M695 t253 nw28 0 0 nch w=1u l=180n
M696 t253 nw42 0 0 nch w=1u l=180n
CT254 t254 0 0.1f
M697 t254 nw28 vdd vdd pch w=2u l=180n
M698 t253 nw42 t254 vdd pch w=2u l=180n
M699 nw96 t253 vdd vdd pch w=2u l=180n
M700 nw96 t253 0 0 nch w=1u l=180n
Cnw96 nw96 0 2f
CT255 t255 0 0.1f
CT256 t256 0 0.1f
CT257 t257 0 0.1f
M701 t255 nw30 vdd vdd pch w=2u l=180n
M702 t255 nw45 vdd vdd pch w=2u l=180n
CT258 t258 0 0.1f
M703 t255 nw30 t258 0 nch w=1u l=180n
M704 t258 nw45 0 0 nch w=1u l=180n
M705 t256 nw30 vdd vdd pch w=2u l=180n
M706 t256 t255 vdd vdd pch w=2u l=180n
CT259 t259 0 0.1f
M707 t256 nw30 t259 0 nch w=1u l=180n
M708 t259 t255 0 0 nch w=1u l=180n
M709 t257 nw45 vdd vdd pch w=2u l=180n
M710 t257 t255 vdd vdd pch w=2u l=180n
CT260 t260 0 0.1f
M711 t257 nw45 t260 0 nch w=1u l=180n
M712 t260 t255 0 0 nch w=1u l=180n
M713 nw97 t256 vdd vdd pch w=2u l=180n
M714 nw97 t257 vdd vdd pch w=2u l=180n
CT261 t261 0 0.1f
M715 nw97 t256 t261 0 nch w=1u l=180n
M716 t261 t257 0 0 nch w=1u l=180n
Cnw97 nw97 0 2f
M717 nw98 nw32 vdd vdd pch w=2u l=180n
M718 nw98 nw48 vdd vdd pch w=2u l=180n
CT262 t262 0 0.1f
M719 nw98 nw32 t262 0 nch w=1u l=180n
M720 t262 nw48 0 0 nch w=1u l=180n
Cnw98 nw98 0 2f
M721 nw99 nw34 0 0 nch w=1u l=180n
M722 nw99 nw51 0 0 nch w=1u l=180n
CT263 t263 0 0.1f
M723 t263 nw34 vdd vdd pch w=2u l=180n
M724 nw99 nw51 t263 vdd pch w=2u l=180n
Cnw99 nw99 0 2f
CT264 t264 0 0.1f
M725 t264 nw36 vdd vdd pch w=2u l=180n
M726 t264 nw54 vdd vdd pch w=2u l=180n
CT265 t265 0 0.1f
M727 t264 nw36 t265 0 nch w=1u l=180n
M728 t265 nw54 0 0 nch w=1u l=180n
M729 nw100 t264 vdd vdd pch w=2u l=180n
M730 nw100 t264 0 0 nch w=1u l=180n
Cnw100 nw100 0 2f
CT266 t266 0 0.1f
M731 t266 nw38 0 0 nch w=1u l=180n
M732 t266 nw57 0 0 nch w=1u l=180n
CT267 t267 0 0.1f
M733 t267 nw38 vdd vdd pch w=2u l=180n
M734 t266 nw57 t267 vdd pch w=2u l=180n
M735 nw101 t266 vdd vdd pch w=2u l=180n
M736 nw101 t266 0 0 nch w=1u l=180n
Cnw101 nw101 0 2f
CT268 t268 0 0.1f
CT269 t269 0 0.1f
CT270 t270 0 0.1f
M737 t268 nw40 vdd vdd pch w=2u l=180n
M738 t268 nw60 vdd vdd pch w=2u l=180n
CT271 t271 0 0.1f
M739 t268 nw40 t271 0 nch w=1u l=180n
M740 t271 nw60 0 0 nch w=1u l=180n
M741 t269 nw40 vdd vdd pch w=2u l=180n
M742 t269 t268 vdd vdd pch w=2u l=180n
CT272 t272 0 0.1f
M743 t269 nw40 t272 0 nch w=1u l=180n
M744 t272 t268 0 0 nch w=1u l=180n
M745 t270 nw60 vdd vdd pch w=2u l=180n
M746 t270 t268 vdd vdd pch w=2u l=180n
CT273 t273 0 0.1f
M747 t270 nw60 t273 0 nch w=1u l=180n
M748 t273 t268 0 0 nch w=1u l=180n
M749 nw102 t269 vdd vdd pch w=2u l=180n
M750 nw102 t270 vdd vdd pch w=2u l=180n
CT274 t274 0 0.1f
M751 nw102 t269 t274 0 nch w=1u l=180n
M752 t274 t270 0 0 nch w=1u l=180n
Cnw102 nw102 0 2f
M753 nw103 nw42 vdd vdd pch w=2u l=180n
M754 nw103 nw63 vdd vdd pch w=2u l=180n
CT275 t275 0 0.1f
M755 nw103 nw42 t275 0 nch w=1u l=180n
M756 t275 nw63 0 0 nch w=1u l=180n
Cnw103 nw103 0 2f
M757 nw104 nw44 0 0 nch w=1u l=180n
M758 nw104 nw66 0 0 nch w=1u l=180n
CT276 t276 0 0.1f
M759 t276 nw44 vdd vdd pch w=2u l=180n
M760 nw104 nw66 t276 vdd pch w=2u l=180n
Cnw104 nw104 0 2f
CT277 t277 0 0.1f
M761 t277 nw46 vdd vdd pch w=2u l=180n
M762 t277 nw69 vdd vdd pch w=2u l=180n
CT278 t278 0 0.1f
M763 t277 nw46 t278 0 nch w=1u l=180n
M764 t278 nw69 0 0 nch w=1u l=180n
M765 nw105 t277 vdd vdd pch w=2u l=180n
M766 nw105 t277 0 0 nch w=1u l=180n
Cnw105 nw105 0 2f
CT279 t279 0 0.1f
M767 t279 nw48 0 0 nch w=1u l=180n
M768 t279 nw72 0 0 nch w=1u l=180n
CT280 t280 0 0.1f
M769 t280 nw48 vdd vdd pch w=2u l=180n
M770 t279 nw72 t280 vdd pch w=2u l=180n
M771 nw106 t279 vdd vdd pch w=2u l=180n
M772 nw106 t279 0 0 nch w=1u l=180n
Cnw106 nw106 0 2f
CT281 t281 0 0.1f
CT282 t282 0 0.1f
CT283 t283 0 0.1f
M773 t281 nw50 vdd vdd pch w=2u l=180n
M774 t281 nw75 vdd vdd pch w=2u l=180n
CT284 t284 0 0.1f
M775 t281 nw50 t284 0 nch w=1u l=180n
M776 t284 nw75 0 0 nch w=1u l=180n
M777 t282 nw50 vdd vdd pch w=2u l=180n
M778 t282 t281 vdd vdd pch w=2u l=180n
CT285 t285 0 0.1f
M779 t282 nw50 t285 0 nch w=1u l=180n
M780 t285 t281 0 0 nch w=1u l=180n
M781 t283 nw75 vdd vdd pch w=2u l=180n
M782 t283 t281 vdd vdd pch w=2u l=180n
CT286 t286 0 0.1f
M783 t283 nw75 t286 0 nch w=1u l=180n
M784 t286 t281 0 0 nch w=1u l=180n
M785 nw107 t282 vdd vdd pch w=2u l=180n
M786 nw107 t283 vdd vdd pch w=2u l=180n
CT287 t287 0 0.1f
M787 nw107 t282 t287 0 nch w=1u l=180n
M788 t287 t283 0 0 nch w=1u l=180n
Cnw107 nw107 0 2f
M789 nw108 nw52 vdd vdd pch w=2u l=180n
M790 nw108 nw78 vdd vdd pch w=2u l=180n
CT288 t288 0 0.1f
M791 nw108 nw52 t288 0 nch w=1u l=180n
M792 t288 nw78 0 0 nch w=1u l=180n
Cnw108 nw108 0 2f
M793 nw109 nw54 0 0 nch w=1u l=180n
M794 nw109 nw81 0 0 nch w=1u l=180n
CT289 t289 0 0.1f
M795 t289 nw54 vdd vdd pch w=2u l=180n
M796 nw109 nw81 t289 vdd pch w=2u l=180n
Cnw109 nw109 0 2f
CT290 t290 0 0.1f
M797 t290 nw56 vdd vdd pch w=2u l=180n
M798 t290 nw84 vdd vdd pch w=2u l=180n
CT291 t291 0 0.1f
M799 t290 nw56 t291 0 nch w=1u l=180n
M800 t291 nw84 0 0 nch w=1u l=180n
M801 nw110 t290 vdd vdd pch w=2u l=180n
M802 nw110 t290 0 0 nch w=1u l=180n
Cnw110 nw110 0 2f
CT292 t292 0 0.1f
M803 t292 nw58 0 0 nch w=1u l=180n
M804 t292 nw87 0 0 nch w=1u l=180n
CT293 t293 0 0.1f
M805 t293 nw58 vdd vdd pch w=2u l=180n
M806 t292 nw87 t293 vdd pch w=2u l=180n
M807 nw111 t292 vdd vdd pch w=2u l=180n
M808 nw111 t292 0 0 nch w=1u l=180n
Cnw111 nw111 0 2f
CT294 t294 0 0.1f
CT295 t295 0 0.1f
CT296 t296 0 0.1f
M809 t294 nw60 vdd vdd pch w=2u l=180n
M810 t294 nw90 vdd vdd pch w=2u l=180n
CT297 t297 0 0.1f
M811 t294 nw60 t297 0 nch w=1u l=180n
M812 t297 nw90 0 0 nch w=1u l=180n
M813 t295 nw60 vdd vdd pch w=2u l=180n
M814 t295 t294 vdd vdd pch w=2u l=180n
CT298 t298 0 0.1f
M815 t295 nw60 t298 0 nch w=1u l=180n
M816 t298 t294 0 0 nch w=1u l=180n
M817 t296 nw90 vdd vdd pch w=2u l=180n
M818 t296 t294 vdd vdd pch w=2u l=180n
CT299 t299 0 0.1f
M819 t296 nw90 t299 0 nch w=1u l=180n
M820 t299 t294 0 0 nch w=1u l=180n
M821 nw112 t295 vdd vdd pch w=2u l=180n
M822 nw112 t296 vdd vdd pch w=2u l=180n
CT300 t300 0 0.1f
M823 nw112 t295 t300 0 nch w=1u l=180n
M824 t300 t296 0 0 nch w=1u l=180n
Cnw112 nw112 0 2f
M825 nw113 nw62 vdd vdd pch w=2u l=180n
M826 nw113 nw93 vdd vdd pch w=2u l=180n
CT301 t301 0 0.1f
M827 nw113 nw62 t301 0 nch w=1u l=180n
M828 t301 nw93 0 0 nch w=1u l=180n
Cnw113 nw113 0 2f
M829 nw114 nw64 0 0 nch w=1u l=180n
M830 nw114 nw96 0 0 nch w=1u l=180n
CT302 t302 0 0.1f
M831 t302 nw64 vdd vdd pch w=2u l=180n
M832 nw114 nw96 t302 vdd pch w=2u l=180n
Cnw114 nw114 0 2f
CT303 t303 0 0.1f
M833 t303 nw66 vdd vdd pch w=2u l=180n
M834 t303 nw99 vdd vdd pch w=2u l=180n
CT304 t304 0 0.1f
M835 t303 nw66 t304 0 nch w=1u l=180n
M836 t304 nw99 0 0 nch w=1u l=180n
M837 nw115 t303 vdd vdd pch w=2u l=180n
M838 nw115 t303 0 0 nch w=1u l=180n
Cnw115 nw115 0 2f
CT305 t305 0 0.1f
M839 t305 nw68 0 0 nch w=1u l=180n
M840 t305 nw102 0 0 nch w=1u l=180n
CT306 t306 0 0.1f
M841 t306 nw68 vdd vdd pch w=2u l=180n
M842 t305 nw102 t306 vdd pch w=2u l=180n
M843 nw116 t305 vdd vdd pch w=2u l=180n
M844 nw116 t305 0 0 nch w=1u l=180n
Cnw116 nw116 0 2f
CT307 t307 0 0.1f
CT308 t308 0 0.1f
CT309 t309 0 0.1f
M845 t307 nw70 vdd vdd pch w=2u l=180n
M846 t307 nw105 vdd vdd pch w=2u l=180n
CT310 t310 0 0.1f
M847 t307 nw70 t310 0 nch w=1u l=180n
M848 t310 nw105 0 0 nch w=1u l=180n
M849 t308 nw70 vdd vdd pch w=2u l=180n
M850 t308 t307 vdd vdd pch w=2u l=180n
CT311 t311 0 0.1f
M851 t308 nw70 t311 0 nch w=1u l=180n
M852 t311 t307 0 0 nch w=1u l=180n
M853 t309 nw105 vdd vdd pch w=2u l=180n
M854 t309 t307 vdd vdd pch w=2u l=180n
CT312 t312 0 0.1f
M855 t309 nw105 t312 0 nch w=1u l=180n
M856 t312 t307 0 0 nch w=1u l=180n
M857 nw117 t308 vdd vdd pch w=2u l=180n
M858 nw117 t309 vdd vdd pch w=2u l=180n
CT313 t313 0 0.1f
M859 nw117 t308 t313 0 nch w=1u l=180n
M860 t313 t309 0 0 nch w=1u l=180n
Cnw117 nw117 0 2f
M861 nw118 nw72 vdd vdd pch w=2u l=180n
M862 nw118 nw108 vdd vdd pch w=2u l=180n
CT314 t314 0 0.1f
M863 nw118 nw72 t314 0 nch w=1u l=180n
M864 t314 nw108 0 0 nch w=1u l=180n
Cnw118 nw118 0 2f
M865 nw119 nw74 0 0 nch w=1u l=180n
M866 nw119 nw111 0 0 nch w=1u l=180n
CT315 t315 0 0.1f
M867 t315 nw74 vdd vdd pch w=2u l=180n
M868 nw119 nw111 t315 vdd pch w=2u l=180n
Cnw119 nw119 0 2f
CT316 t316 0 0.1f
M869 t316 nw76 vdd vdd pch w=2u l=180n
M870 t316 nw114 vdd vdd pch w=2u l=180n
CT317 t317 0 0.1f
M871 t316 nw76 t317 0 nch w=1u l=180n
M872 t317 nw114 0 0 nch w=1u l=180n
M873 nw120 t316 vdd vdd pch w=2u l=180n
M874 nw120 t316 0 0 nch w=1u l=180n
Cnw120 nw120 0 2f
CT318 t318 0 0.1f
M875 t318 nw78 0 0 nch w=1u l=180n
M876 t318 nw117 0 0 nch w=1u l=180n
CT319 t319 0 0.1f
M877 t319 nw78 vdd vdd pch w=2u l=180n
M878 t318 nw117 t319 vdd pch w=2u l=180n
M879 nw121 t318 vdd vdd pch w=2u l=180n
M880 nw121 t318 0 0 nch w=1u l=180n
Cnw121 nw121 0 2f
CT320 t320 0 0.1f
CT321 t321 0 0.1f
CT322 t322 0 0.1f
M881 t320 nw80 vdd vdd pch w=2u l=180n
M882 t320 nw120 vdd vdd pch w=2u l=180n
CT323 t323 0 0.1f
M883 t320 nw80 t323 0 nch w=1u l=180n
M884 t323 nw120 0 0 nch w=1u l=180n
M885 t321 nw80 vdd vdd pch w=2u l=180n
M886 t321 t320 vdd vdd pch w=2u l=180n
CT324 t324 0 0.1f
M887 t321 nw80 t324 0 nch w=1u l=180n
M888 t324 t320 0 0 nch w=1u l=180n
M889 t322 nw120 vdd vdd pch w=2u l=180n
M890 t322 t320 vdd vdd pch w=2u l=180n
CT325 t325 0 0.1f
M891 t322 nw120 t325 0 nch w=1u l=180n
M892 t325 t320 0 0 nch w=1u l=180n
M893 nw122 t321 vdd vdd pch w=2u l=180n
M894 nw122 t322 vdd vdd pch w=2u l=180n
CT326 t326 0 0.1f
M895 nw122 t321 t326 0 nch w=1u l=180n
M896 t326 t322 0 0 nch w=1u l=180n
Cnw122 nw122 0 2f
M897 nw123 nw82 vdd vdd pch w=2u l=180n
M898 nw123 nq0 vdd vdd pch w=2u l=180n
CT327 t327 0 0.1f
M899 nw123 nw82 t327 0 nch w=1u l=180n
M900 t327 nq0 0 0 nch w=1u l=180n
Cnw123 nw123 0 2f
M901 nw124 nw84 0 0 nch w=1u l=180n
M902 nw124 nq2 0 0 nch w=1u l=180n
CT328 t328 0 0.1f
M903 t328 nw84 vdd vdd pch w=2u l=180n
M904 nw124 nq2 t328 vdd pch w=2u l=180n
Cnw124 nw124 0 2f
CT329 t329 0 0.1f
M905 t329 nw86 vdd vdd pch w=2u l=180n
M906 t329 nq4 vdd vdd pch w=2u l=180n
CT330 t330 0 0.1f
M907 t329 nw86 t330 0 nch w=1u l=180n
M908 t330 nq4 0 0 nch w=1u l=180n
M909 nw125 t329 vdd vdd pch w=2u l=180n
M910 nw125 t329 0 0 nch w=1u l=180n
Cnw125 nw125 0 2f
CT331 t331 0 0.1f
M911 t331 nw88 0 0 nch w=1u l=180n
M912 t331 nq6 0 0 nch w=1u l=180n
CT332 t332 0 0.1f
M913 t332 nw88 vdd vdd pch w=2u l=180n
M914 t331 nq6 t332 vdd pch w=2u l=180n
M915 nw126 t331 vdd vdd pch w=2u l=180n
M916 nw126 t331 0 0 nch w=1u l=180n
Cnw126 nw126 0 2f
CT333 t333 0 0.1f
CT334 t334 0 0.1f
CT335 t335 0 0.1f
M917 t333 nw90 vdd vdd pch w=2u l=180n
M918 t333 nq8 vdd vdd pch w=2u l=180n
CT336 t336 0 0.1f
M919 t333 nw90 t336 0 nch w=1u l=180n
M920 t336 nq8 0 0 nch w=1u l=180n
M921 t334 nw90 vdd vdd pch w=2u l=180n
M922 t334 t333 vdd vdd pch w=2u l=180n
CT337 t337 0 0.1f
M923 t334 nw90 t337 0 nch w=1u l=180n
M924 t337 t333 0 0 nch w=1u l=180n
M925 t335 nq8 vdd vdd pch w=2u l=180n
M926 t335 t333 vdd vdd pch w=2u l=180n
CT338 t338 0 0.1f
M927 t335 nq8 t338 0 nch w=1u l=180n
M928 t338 t333 0 0 nch w=1u l=180n
M929 nw127 t334 vdd vdd pch w=2u l=180n
M930 nw127 t335 vdd vdd pch w=2u l=180n
CT339 t339 0 0.1f
M931 nw127 t334 t339 0 nch w=1u l=180n
M932 t339 t335 0 0 nch w=1u l=180n
Cnw127 nw127 0 2f
M933 nw128 nw92 vdd vdd pch w=2u l=180n
M934 nw128 nq10 vdd vdd pch w=2u l=180n
CT340 t340 0 0.1f
M935 nw128 nw92 t340 0 nch w=1u l=180n
M936 t340 nq10 0 0 nch w=1u l=180n
Cnw128 nw128 0 2f
M937 nw129 nw94 0 0 nch w=1u l=180n
M938 nw129 nq12 0 0 nch w=1u l=180n
CT341 t341 0 0.1f
M939 t341 nw94 vdd vdd pch w=2u l=180n
M940 nw129 nq12 t341 vdd pch w=2u l=180n
Cnw129 nw129 0 2f
CT342 t342 0 0.1f
M941 t342 nw96 vdd vdd pch w=2u l=180n
M942 t342 nq14 vdd vdd pch w=2u l=180n
CT343 t343 0 0.1f
M943 t342 nw96 t343 0 nch w=1u l=180n
M944 t343 nq14 0 0 nch w=1u l=180n
M945 nw130 t342 vdd vdd pch w=2u l=180n
M946 nw130 t342 0 0 nch w=1u l=180n
Cnw130 nw130 0 2f
CT344 t344 0 0.1f
M947 t344 nw98 0 0 nch w=1u l=180n
M948 t344 nq16 0 0 nch w=1u l=180n
CT345 t345 0 0.1f
M949 t345 nw98 vdd vdd pch w=2u l=180n
M950 t344 nq16 t345 vdd pch w=2u l=180n
M951 nw131 t344 vdd vdd pch w=2u l=180n
M952 nw131 t344 0 0 nch w=1u l=180n
Cnw131 nw131 0 2f
CT346 t346 0 0.1f
CT347 t347 0 0.1f
CT348 t348 0 0.1f
M953 t346 nw100 vdd vdd pch w=2u l=180n
M954 t346 ni0 vdd vdd pch w=2u l=180n
CT349 t349 0 0.1f
M955 t346 nw100 t349 0 nch w=1u l=180n
M956 t349 ni0 0 0 nch w=1u l=180n
M957 t347 nw100 vdd vdd pch w=2u l=180n
M958 t347 t346 vdd vdd pch w=2u l=180n
CT350 t350 0 0.1f
M959 t347 nw100 t350 0 nch w=1u l=180n
M960 t350 t346 0 0 nch w=1u l=180n
M961 t348 ni0 vdd vdd pch w=2u l=180n
M962 t348 t346 vdd vdd pch w=2u l=180n
CT351 t351 0 0.1f
M963 t348 ni0 t351 0 nch w=1u l=180n
M964 t351 t346 0 0 nch w=1u l=180n
M965 nw132 t347 vdd vdd pch w=2u l=180n
M966 nw132 t348 vdd vdd pch w=2u l=180n
CT352 t352 0 0.1f
M967 nw132 t347 t352 0 nch w=1u l=180n
M968 t352 t348 0 0 nch w=1u l=180n
Cnw132 nw132 0 2f
M969 nw133 nw102 vdd vdd pch w=2u l=180n
M970 nw133 ni2 vdd vdd pch w=2u l=180n
CT353 t353 0 0.1f
M971 nw133 nw102 t353 0 nch w=1u l=180n
M972 t353 ni2 0 0 nch w=1u l=180n
Cnw133 nw133 0 2f
M973 nw134 nw104 0 0 nch w=1u l=180n
M974 nw134 ni4 0 0 nch w=1u l=180n
CT354 t354 0 0.1f
M975 t354 nw104 vdd vdd pch w=2u l=180n
M976 nw134 ni4 t354 vdd pch w=2u l=180n
Cnw134 nw134 0 2f
CT355 t355 0 0.1f
M977 t355 nw106 vdd vdd pch w=2u l=180n
M978 t355 ni6 vdd vdd pch w=2u l=180n
CT356 t356 0 0.1f
M979 t355 nw106 t356 0 nch w=1u l=180n
M980 t356 ni6 0 0 nch w=1u l=180n
M981 nw135 t355 vdd vdd pch w=2u l=180n
M982 nw135 t355 0 0 nch w=1u l=180n
Cnw135 nw135 0 2f
CT357 t357 0 0.1f
M983 t357 nw108 0 0 nch w=1u l=180n
M984 t357 ni8 0 0 nch w=1u l=180n
CT358 t358 0 0.1f
M985 t358 nw108 vdd vdd pch w=2u l=180n
M986 t357 ni8 t358 vdd pch w=2u l=180n
M987 nw136 t357 vdd vdd pch w=2u l=180n
M988 nw136 t357 0 0 nch w=1u l=180n
Cnw136 nw136 0 2f
CT359 t359 0 0.1f
CT360 t360 0 0.1f
CT361 t361 0 0.1f
M989 t359 nw110 vdd vdd pch w=2u l=180n
M990 t359 nw4 vdd vdd pch w=2u l=180n
CT362 t362 0 0.1f
M991 t359 nw110 t362 0 nch w=1u l=180n
M992 t362 nw4 0 0 nch w=1u l=180n
M993 t360 nw110 vdd vdd pch w=2u l=180n
M994 t360 t359 vdd vdd pch w=2u l=180n
CT363 t363 0 0.1f
M995 t360 nw110 t363 0 nch w=1u l=180n
M996 t363 t359 0 0 nch w=1u l=180n
M997 t361 nw4 vdd vdd pch w=2u l=180n
M998 t361 t359 vdd vdd pch w=2u l=180n
CT364 t364 0 0.1f
M999 t361 nw4 t364 0 nch w=1u l=180n
M1000 t364 t359 0 0 nch w=1u l=180n
M1001 nw137 t360 vdd vdd pch w=2u l=180n
M1002 nw137 t361 vdd vdd pch w=2u l=180n
CT365 t365 0 0.1f
M1003 nw137 t360 t365 0 nch w=1u l=180n
M1004 t365 t361 0 0 nch w=1u l=180n
Cnw137 nw137 0 2f
M1005 nw138 nw112 vdd vdd pch w=2u l=180n
M1006 nw138 nw6 vdd vdd pch w=2u l=180n
CT366 t366 0 0.1f
M1007 nw138 nw112 t366 0 nch w=1u l=180n
M1008 t366 nw6 0 0 nch w=1u l=180n
Cnw138 nw138 0 2f
M1009 nw139 nw114 0 0 nch w=1u l=180n
M1010 nw139 nw8 0 0 nch w=1u l=180n
CT367 t367 0 0.1f
M1011 t367 nw114 vdd vdd pch w=2u l=180n
M1012 nw139 nw8 t367 vdd pch w=2u l=180n
Cnw139 nw139 0 2f
CT368 t368 0 0.1f
M1013 t368 nw116 vdd vdd pch w=2u l=180n
M1014 t368 nw10 vdd vdd pch w=2u l=180n
CT369 t369 0 0.1f
M1015 t368 nw116 t369 0 nch w=1u l=180n
M1016 t369 nw10 0 0 nch w=1u l=180n
M1017 nw140 t368 vdd vdd pch w=2u l=180n
M1018 nw140 t368 0 0 nch w=1u l=180n
Cnw140 nw140 0 2f
CT370 t370 0 0.1f
M1019 t370 nw118 0 0 nch w=1u l=180n
M1020 t370 nw12 0 0 nch w=1u l=180n
CT371 t371 0 0.1f
M1021 t371 nw118 vdd vdd pch w=2u l=180n
M1022 t370 nw12 t371 vdd pch w=2u l=180n
M1023 nw141 t370 vdd vdd pch w=2u l=180n
M1024 nw141 t370 0 0 nch w=1u l=180n
Cnw141 nw141 0 2f
CT372 t372 0 0.1f
CT373 t373 0 0.1f
CT374 t374 0 0.1f
M1025 t372 nw120 vdd vdd pch w=2u l=180n
M1026 t372 nw14 vdd vdd pch w=2u l=180n
CT375 t375 0 0.1f
M1027 t372 nw120 t375 0 nch w=1u l=180n
M1028 t375 nw14 0 0 nch w=1u l=180n
M1029 t373 nw120 vdd vdd pch w=2u l=180n
M1030 t373 t372 vdd vdd pch w=2u l=180n
CT376 t376 0 0.1f
M1031 t373 nw120 t376 0 nch w=1u l=180n
M1032 t376 t372 0 0 nch w=1u l=180n
M1033 t374 nw14 vdd vdd pch w=2u l=180n
M1034 t374 t372 vdd vdd pch w=2u l=180n
CT377 t377 0 0.1f
M1035 t374 nw14 t377 0 nch w=1u l=180n
M1036 t377 t372 0 0 nch w=1u l=180n
M1037 nw142 t373 vdd vdd pch w=2u l=180n
M1038 nw142 t374 vdd vdd pch w=2u l=180n
CT378 t378 0 0.1f
M1039 nw142 t373 t378 0 nch w=1u l=180n
M1040 t378 t374 0 0 nch w=1u l=180n
Cnw142 nw142 0 2f
M1041 nw143 nw122 vdd vdd pch w=2u l=180n
M1042 nw143 nw16 vdd vdd pch w=2u l=180n
CT379 t379 0 0.1f
M1043 nw143 nw122 t379 0 nch w=1u l=180n
M1044 t379 nw16 0 0 nch w=1u l=180n
Cnw143 nw143 0 2f
M1045 nw144 nw124 0 0 nch w=1u l=180n
M1046 nw144 nw18 0 0 nch w=1u l=180n
CT380 t380 0 0.1f
M1047 t380 nw124 vdd vdd pch w=2u l=180n
M1048 nw144 nw18 t380 vdd pch w=2u l=180n
Cnw144 nw144 0 2f
CT381 t381 0 0.1f
M1049 t381 nw126 vdd vdd pch w=2u l=180n
M1050 t381 nw20 vdd vdd pch w=2u l=180n
CT382 t382 0 0.1f
M1051 t381 nw126 t382 0 nch w=1u l=180n
M1052 t382 nw20 0 0 nch w=1u l=180n
M1053 nw145 t381 vdd vdd pch w=2u l=180n
M1054 nw145 t381 0 0 nch w=1u l=180n
Cnw145 nw145 0 2f
CT383 t383 0 0.1f
M1055 t383 nw128 0 0 nch w=1u l=180n
M1056 t383 nw22 0 0 nch w=1u l=180n
CT384 t384 0 0.1f
M1057 t384 nw128 vdd vdd pch w=2u l=180n
M1058 t383 nw22 t384 vdd pch w=2u l=180n
M1059 nw146 t383 vdd vdd pch w=2u l=180n
M1060 nw146 t383 0 0 nch w=1u l=180n
Cnw146 nw146 0 2f
CT385 t385 0 0.1f
CT386 t386 0 0.1f
CT387 t387 0 0.1f
M1061 t385 nw130 vdd vdd pch w=2u l=180n
M1062 t385 nw24 vdd vdd pch w=2u l=180n
CT388 t388 0 0.1f
M1063 t385 nw130 t388 0 nch w=1u l=180n
M1064 t388 nw24 0 0 nch w=1u l=180n
M1065 t386 nw130 vdd vdd pch w=2u l=180n
M1066 t386 t385 vdd vdd pch w=2u l=180n
CT389 t389 0 0.1f
M1067 t386 nw130 t389 0 nch w=1u l=180n
M1068 t389 t385 0 0 nch w=1u l=180n
M1069 t387 nw24 vdd vdd pch w=2u l=180n
M1070 t387 t385 vdd vdd pch w=2u l=180n
CT390 t390 0 0.1f
M1071 t387 nw24 t390 0 nch w=1u l=180n
M1072 t390 t385 0 0 nch w=1u l=180n
M1073 nw147 t386 vdd vdd pch w=2u l=180n
M1074 nw147 t387 vdd vdd pch w=2u l=180n
CT391 t391 0 0.1f
M1075 nw147 t386 t391 0 nch w=1u l=180n
M1076 t391 t387 0 0 nch w=1u l=180n
Cnw147 nw147 0 2f
M1077 nw148 nw132 vdd vdd pch w=2u l=180n
M1078 nw148 nw26 vdd vdd pch w=2u l=180n
CT392 t392 0 0.1f
M1079 nw148 nw132 t392 0 nch w=1u l=180n
M1080 t392 nw26 0 0 nch w=1u l=180n
Cnw148 nw148 0 2f
M1081 nw149 nw134 0 0 nch w=1u l=180n
M1082 nw149 nw28 0 0 nch w=1u l=180n
CT393 t393 0 0.1f
M1083 t393 nw134 vdd vdd pch w=2u l=180n
M1084 nw149 nw28 t393 vdd pch w=2u l=180n
Cnw149 nw149 0 2f
CT394 t394 0 0.1f
M1085 t394 nw136 vdd vdd pch w=2u l=180n
M1086 t394 nw30 vdd vdd pch w=2u l=180n
CT395 t395 0 0.1f
M1087 t394 nw136 t395 0 nch w=1u l=180n
M1088 t395 nw30 0 0 nch w=1u l=180n
M1089 nw150 t394 vdd vdd pch w=2u l=180n
M1090 nw150 t394 0 0 nch w=1u l=180n
Cnw150 nw150 0 2f
CT396 t396 0 0.1f
M1091 t396 nw138 0 0 nch w=1u l=180n
M1092 t396 nw32 0 0 nch w=1u l=180n
CT397 t397 0 0.1f
M1093 t397 nw138 vdd vdd pch w=2u l=180n
M1094 t396 nw32 t397 vdd pch w=2u l=180n
M1095 nw151 t396 vdd vdd pch w=2u l=180n
M1096 nw151 t396 0 0 nch w=1u l=180n
Cnw151 nw151 0 2f
CT398 t398 0 0.1f
CT399 t399 0 0.1f
CT400 t400 0 0.1f
M1097 t398 nw140 vdd vdd pch w=2u l=180n
M1098 t398 nw34 vdd vdd pch w=2u l=180n
CT401 t401 0 0.1f
M1099 t398 nw140 t401 0 nch w=1u l=180n
M1100 t401 nw34 0 0 nch w=1u l=180n
M1101 t399 nw140 vdd vdd pch w=2u l=180n
M1102 t399 t398 vdd vdd pch w=2u l=180n
CT402 t402 0 0.1f
M1103 t399 nw140 t402 0 nch w=1u l=180n
M1104 t402 t398 0 0 nch w=1u l=180n
M1105 t400 nw34 vdd vdd pch w=2u l=180n
M1106 t400 t398 vdd vdd pch w=2u l=180n
CT403 t403 0 0.1f
M1107 t400 nw34 t403 0 nch w=1u l=180n
M1108 t403 t398 0 0 nch w=1u l=180n
M1109 nw152 t399 vdd vdd pch w=2u l=180n
M1110 nw152 t400 vdd vdd pch w=2u l=180n
CT404 t404 0 0.1f
M1111 nw152 t399 t404 0 nch w=1u l=180n
M1112 t404 t400 0 0 nch w=1u l=180n
Cnw152 nw152 0 2f
M1113 nw153 nw142 vdd vdd pch w=2u l=180n
M1114 nw153 nw36 vdd vdd pch w=2u l=180n
CT405 t405 0 0.1f
M1115 nw153 nw142 t405 0 nch w=1u l=180n
M1116 t405 nw36 0 0 nch w=1u l=180n
Cnw153 nw153 0 2f
M1117 nw154 nw144 0 0 nch w=1u l=180n
M1118 nw154 nw38 0 0 nch w=1u l=180n
CT406 t406 0 0.1f
M1119 t406 nw144 vdd vdd pch w=2u l=180n
M1120 nw154 nw38 t406 vdd pch w=2u l=180n
Cnw154 nw154 0 2f
CT407 t407 0 0.1f
M1121 t407 nw146 vdd vdd pch w=2u l=180n
M1122 t407 nw40 vdd vdd pch w=2u l=180n
CT408 t408 0 0.1f
M1123 t407 nw146 t408 0 nch w=1u l=180n
M1124 t408 nw40 0 0 nch w=1u l=180n
M1125 nw155 t407 vdd vdd pch w=2u l=180n
M1126 nw155 t407 0 0 nch w=1u l=180n
Cnw155 nw155 0 2f
CT409 t409 0 0.1f
M1127 t409 nw148 0 0 nch w=1u l=180n
M1128 t409 nw42 0 0 nch w=1u l=180n
CT410 t410 0 0.1f
M1129 t410 nw148 vdd vdd pch w=2u l=180n
M1130 t409 nw42 t410 vdd pch w=2u l=180n
M1131 nw156 t409 vdd vdd pch w=2u l=180n
M1132 nw156 t409 0 0 nch w=1u l=180n
Cnw156 nw156 0 2f
CT411 t411 0 0.1f
CT412 t412 0 0.1f
CT413 t413 0 0.1f
M1133 t411 nw150 vdd vdd pch w=2u l=180n
M1134 t411 nw44 vdd vdd pch w=2u l=180n
CT414 t414 0 0.1f
M1135 t411 nw150 t414 0 nch w=1u l=180n
M1136 t414 nw44 0 0 nch w=1u l=180n
M1137 t412 nw150 vdd vdd pch w=2u l=180n
M1138 t412 t411 vdd vdd pch w=2u l=180n
CT415 t415 0 0.1f
M1139 t412 nw150 t415 0 nch w=1u l=180n
M1140 t415 t411 0 0 nch w=1u l=180n
M1141 t413 nw44 vdd vdd pch w=2u l=180n
M1142 t413 t411 vdd vdd pch w=2u l=180n
CT416 t416 0 0.1f
M1143 t413 nw44 t416 0 nch w=1u l=180n
M1144 t416 t411 0 0 nch w=1u l=180n
M1145 nw157 t412 vdd vdd pch w=2u l=180n
M1146 nw157 t413 vdd vdd pch w=2u l=180n
CT417 t417 0 0.1f
M1147 nw157 t412 t417 0 nch w=1u l=180n
M1148 t417 t413 0 0 nch w=1u l=180n
Cnw157 nw157 0 2f
M1149 nw158 nw152 vdd vdd pch w=2u l=180n
M1150 nw158 nw46 vdd vdd pch w=2u l=180n
CT418 t418 0 0.1f
M1151 nw158 nw152 t418 0 nch w=1u l=180n
M1152 t418 nw46 0 0 nch w=1u l=180n
Cnw158 nw158 0 2f
M1153 nw159 nw154 0 0 nch w=1u l=180n
M1154 nw159 nw48 0 0 nch w=1u l=180n
CT419 t419 0 0.1f
M1155 t419 nw154 vdd vdd pch w=2u l=180n
M1156 nw159 nw48 t419 vdd pch w=2u l=180n
Cnw159 nw159 0 2f
CT420 t420 0 0.1f
M1157 t420 nw156 vdd vdd pch w=2u l=180n
M1158 t420 nw50 vdd vdd pch w=2u l=180n
CT421 t421 0 0.1f
M1159 t420 nw156 t421 0 nch w=1u l=180n
M1160 t421 nw50 0 0 nch w=1u l=180n
M1161 nw160 t420 vdd vdd pch w=2u l=180n
M1162 nw160 t420 0 0 nch w=1u l=180n
Cnw160 nw160 0 2f
CT422 t422 0 0.1f
M1163 t422 nw158 0 0 nch w=1u l=180n
M1164 t422 nw52 0 0 nch w=1u l=180n
CT423 t423 0 0.1f
M1165 t423 nw158 vdd vdd pch w=2u l=180n
M1166 t422 nw52 t423 vdd pch w=2u l=180n
M1167 nw161 t422 vdd vdd pch w=2u l=180n
M1168 nw161 t422 0 0 nch w=1u l=180n
Cnw161 nw161 0 2f
CT424 t424 0 0.1f
CT425 t425 0 0.1f
CT426 t426 0 0.1f
M1169 t424 nw160 vdd vdd pch w=2u l=180n
M1170 t424 nw54 vdd vdd pch w=2u l=180n
CT427 t427 0 0.1f
M1171 t424 nw160 t427 0 nch w=1u l=180n
M1172 t427 nw54 0 0 nch w=1u l=180n
M1173 t425 nw160 vdd vdd pch w=2u l=180n
M1174 t425 t424 vdd vdd pch w=2u l=180n
CT428 t428 0 0.1f
M1175 t425 nw160 t428 0 nch w=1u l=180n
M1176 t428 t424 0 0 nch w=1u l=180n
M1177 t426 nw54 vdd vdd pch w=2u l=180n
M1178 t426 t424 vdd vdd pch w=2u l=180n
CT429 t429 0 0.1f
M1179 t426 nw54 t429 0 nch w=1u l=180n
M1180 t429 t424 0 0 nch w=1u l=180n
M1181 nw162 t425 vdd vdd pch w=2u l=180n
M1182 nw162 t426 vdd vdd pch w=2u l=180n
CT430 t430 0 0.1f
M1183 nw162 t425 t430 0 nch w=1u l=180n
M1184 t430 t426 0 0 nch w=1u l=180n
Cnw162 nw162 0 2f
M1185 nw163 nw162 vdd vdd pch w=2u l=180n
M1186 nw163 nw56 vdd vdd pch w=2u l=180n
CT431 t431 0 0.1f
M1187 nw163 nw162 t431 0 nch w=1u l=180n
M1188 t431 nw56 0 0 nch w=1u l=180n
Cnw163 nw163 0 2f
M1189 nw164 nq0 0 0 nch w=1u l=180n
M1190 nw164 nw58 0 0 nch w=1u l=180n
CT432 t432 0 0.1f
M1191 t432 nq0 vdd vdd pch w=2u l=180n
M1192 nw164 nw58 t432 vdd pch w=2u l=180n
Cnw164 nw164 0 2f
CT433 t433 0 0.1f
M1193 t433 nq1 vdd vdd pch w=2u l=180n
M1194 t433 nw60 vdd vdd pch w=2u l=180n
CT434 t434 0 0.1f
M1195 t433 nq1 t434 0 nch w=1u l=180n
M1196 t434 nw60 0 0 nch w=1u l=180n
M1197 nw165 t433 vdd vdd pch w=2u l=180n
M1198 nw165 t433 0 0 nch w=1u l=180n
Cnw165 nw165 0 2f
CT435 t435 0 0.1f
M1199 t435 nq2 0 0 nch w=1u l=180n
M1200 t435 nw62 0 0 nch w=1u l=180n
CT436 t436 0 0.1f
M1201 t436 nq2 vdd vdd pch w=2u l=180n
M1202 t435 nw62 t436 vdd pch w=2u l=180n
M1203 nw166 t435 vdd vdd pch w=2u l=180n
M1204 nw166 t435 0 0 nch w=1u l=180n
Cnw166 nw166 0 2f
CT437 t437 0 0.1f
CT438 t438 0 0.1f
CT439 t439 0 0.1f
M1205 t437 nq3 vdd vdd pch w=2u l=180n
M1206 t437 nw64 vdd vdd pch w=2u l=180n
CT440 t440 0 0.1f
M1207 t437 nq3 t440 0 nch w=1u l=180n
M1208 t440 nw64 0 0 nch w=1u l=180n
M1209 t438 nq3 vdd vdd pch w=2u l=180n
M1210 t438 t437 vdd vdd pch w=2u l=180n
CT441 t441 0 0.1f
M1211 t438 nq3 t441 0 nch w=1u l=180n
M1212 t441 t437 0 0 nch w=1u l=180n
M1213 t439 nw64 vdd vdd pch w=2u l=180n
M1214 t439 t437 vdd vdd pch w=2u l=180n
CT442 t442 0 0.1f
M1215 t439 nw64 t442 0 nch w=1u l=180n
M1216 t442 t437 0 0 nch w=1u l=180n
M1217 nw167 t438 vdd vdd pch w=2u l=180n
M1218 nw167 t439 vdd vdd pch w=2u l=180n
CT443 t443 0 0.1f
M1219 nw167 t438 t443 0 nch w=1u l=180n
M1220 t443 t439 0 0 nch w=1u l=180n
Cnw167 nw167 0 2f
M1221 nw168 nq4 vdd vdd pch w=2u l=180n
M1222 nw168 nw66 vdd vdd pch w=2u l=180n
CT444 t444 0 0.1f
M1223 nw168 nq4 t444 0 nch w=1u l=180n
M1224 t444 nw66 0 0 nch w=1u l=180n
Cnw168 nw168 0 2f
M1225 nw169 nq5 0 0 nch w=1u l=180n
M1226 nw169 nw68 0 0 nch w=1u l=180n
CT445 t445 0 0.1f
M1227 t445 nq5 vdd vdd pch w=2u l=180n
M1228 nw169 nw68 t445 vdd pch w=2u l=180n
Cnw169 nw169 0 2f
CT446 t446 0 0.1f
M1229 t446 nq6 vdd vdd pch w=2u l=180n
M1230 t446 nw70 vdd vdd pch w=2u l=180n
CT447 t447 0 0.1f
M1231 t446 nq6 t447 0 nch w=1u l=180n
M1232 t447 nw70 0 0 nch w=1u l=180n
M1233 nw170 t446 vdd vdd pch w=2u l=180n
M1234 nw170 t446 0 0 nch w=1u l=180n
Cnw170 nw170 0 2f
CT448 t448 0 0.1f
M1235 t448 nq7 0 0 nch w=1u l=180n
M1236 t448 nw72 0 0 nch w=1u l=180n
CT449 t449 0 0.1f
M1237 t449 nq7 vdd vdd pch w=2u l=180n
M1238 t448 nw72 t449 vdd pch w=2u l=180n
M1239 nw171 t448 vdd vdd pch w=2u l=180n
M1240 nw171 t448 0 0 nch w=1u l=180n
Cnw171 nw171 0 2f
CT450 t450 0 0.1f
CT451 t451 0 0.1f
CT452 t452 0 0.1f
M1241 t450 nq8 vdd vdd pch w=2u l=180n
M1242 t450 nw74 vdd vdd pch w=2u l=180n
CT453 t453 0 0.1f
M1243 t450 nq8 t453 0 nch w=1u l=180n
M1244 t453 nw74 0 0 nch w=1u l=180n
M1245 t451 nq8 vdd vdd pch w=2u l=180n
M1246 t451 t450 vdd vdd pch w=2u l=180n
CT454 t454 0 0.1f
M1247 t451 nq8 t454 0 nch w=1u l=180n
M1248 t454 t450 0 0 nch w=1u l=180n
M1249 t452 nw74 vdd vdd pch w=2u l=180n
M1250 t452 t450 vdd vdd pch w=2u l=180n
CT455 t455 0 0.1f
M1251 t452 nw74 t455 0 nch w=1u l=180n
M1252 t455 t450 0 0 nch w=1u l=180n
M1253 nw172 t451 vdd vdd pch w=2u l=180n
M1254 nw172 t452 vdd vdd pch w=2u l=180n
CT456 t456 0 0.1f
M1255 nw172 t451 t456 0 nch w=1u l=180n
M1256 t456 t452 0 0 nch w=1u l=180n
Cnw172 nw172 0 2f
M1257 nw173 nq9 vdd vdd pch w=2u l=180n
M1258 nw173 nw76 vdd vdd pch w=2u l=180n
CT457 t457 0 0.1f
M1259 nw173 nq9 t457 0 nch w=1u l=180n
M1260 t457 nw76 0 0 nch w=1u l=180n
Cnw173 nw173 0 2f
M1261 nw174 nq10 0 0 nch w=1u l=180n
M1262 nw174 nw78 0 0 nch w=1u l=180n
CT458 t458 0 0.1f
M1263 t458 nq10 vdd vdd pch w=2u l=180n
M1264 nw174 nw78 t458 vdd pch w=2u l=180n
Cnw174 nw174 0 2f
CT459 t459 0 0.1f
M1265 t459 nq11 vdd vdd pch w=2u l=180n
M1266 t459 nw80 vdd vdd pch w=2u l=180n
CT460 t460 0 0.1f
M1267 t459 nq11 t460 0 nch w=1u l=180n
M1268 t460 nw80 0 0 nch w=1u l=180n
M1269 nw175 t459 vdd vdd pch w=2u l=180n
M1270 nw175 t459 0 0 nch w=1u l=180n
Cnw175 nw175 0 2f
CT461 t461 0 0.1f
M1271 t461 nq12 0 0 nch w=1u l=180n
M1272 t461 nw82 0 0 nch w=1u l=180n
CT462 t462 0 0.1f
M1273 t462 nq12 vdd vdd pch w=2u l=180n
M1274 t461 nw82 t462 vdd pch w=2u l=180n
M1275 nw176 t461 vdd vdd pch w=2u l=180n
M1276 nw176 t461 0 0 nch w=1u l=180n
Cnw176 nw176 0 2f
CT463 t463 0 0.1f
CT464 t464 0 0.1f
CT465 t465 0 0.1f
M1277 t463 nq13 vdd vdd pch w=2u l=180n
M1278 t463 nw84 vdd vdd pch w=2u l=180n
CT466 t466 0 0.1f
M1279 t463 nq13 t466 0 nch w=1u l=180n
M1280 t466 nw84 0 0 nch w=1u l=180n
M1281 t464 nq13 vdd vdd pch w=2u l=180n
M1282 t464 t463 vdd vdd pch w=2u l=180n
CT467 t467 0 0.1f
M1283 t464 nq13 t467 0 nch w=1u l=180n
M1284 t467 t463 0 0 nch w=1u l=180n
M1285 t465 nw84 vdd vdd pch w=2u l=180n
M1286 t465 t463 vdd vdd pch w=2u l=180n
CT468 t468 0 0.1f
M1287 t465 nw84 t468 0 nch w=1u l=180n
M1288 t468 t463 0 0 nch w=1u l=180n
M1289 nw177 t464 vdd vdd pch w=2u l=180n
M1290 nw177 t465 vdd vdd pch w=2u l=180n
CT469 t469 0 0.1f
M1291 nw177 t464 t469 0 nch w=1u l=180n
M1292 t469 t465 0 0 nch w=1u l=180n
Cnw177 nw177 0 2f
M1293 nw178 nq14 vdd vdd pch w=2u l=180n
M1294 nw178 nw86 vdd vdd pch w=2u l=180n
CT470 t470 0 0.1f
M1295 nw178 nq14 t470 0 nch w=1u l=180n
M1296 t470 nw86 0 0 nch w=1u l=180n
Cnw178 nw178 0 2f
M1297 nw179 nq15 0 0 nch w=1u l=180n
M1298 nw179 nw88 0 0 nch w=1u l=180n
CT471 t471 0 0.1f
M1299 t471 nq15 vdd vdd pch w=2u l=180n
M1300 nw179 nw88 t471 vdd pch w=2u l=180n
Cnw179 nw179 0 2f
CT472 t472 0 0.1f
M1301 t472 nq16 vdd vdd pch w=2u l=180n
M1302 t472 nw90 vdd vdd pch w=2u l=180n
CT473 t473 0 0.1f
M1303 t472 nq16 t473 0 nch w=1u l=180n
M1304 t473 nw90 0 0 nch w=1u l=180n
M1305 nw180 t472 vdd vdd pch w=2u l=180n
M1306 nw180 t472 0 0 nch w=1u l=180n
Cnw180 nw180 0 2f
CT474 t474 0 0.1f
M1307 t474 nq17 0 0 nch w=1u l=180n
M1308 t474 nw92 0 0 nch w=1u l=180n
CT475 t475 0 0.1f
M1309 t475 nq17 vdd vdd pch w=2u l=180n
M1310 t474 nw92 t475 vdd pch w=2u l=180n
M1311 nw181 t474 vdd vdd pch w=2u l=180n
M1312 nw181 t474 0 0 nch w=1u l=180n
Cnw181 nw181 0 2f
CT476 t476 0 0.1f
CT477 t477 0 0.1f
CT478 t478 0 0.1f
M1313 t476 ni0 vdd vdd pch w=2u l=180n
M1314 t476 nw94 vdd vdd pch w=2u l=180n
CT479 t479 0 0.1f
M1315 t476 ni0 t479 0 nch w=1u l=180n
M1316 t479 nw94 0 0 nch w=1u l=180n
M1317 t477 ni0 vdd vdd pch w=2u l=180n
M1318 t477 t476 vdd vdd pch w=2u l=180n
CT480 t480 0 0.1f
M1319 t477 ni0 t480 0 nch w=1u l=180n
M1320 t480 t476 0 0 nch w=1u l=180n
M1321 t478 nw94 vdd vdd pch w=2u l=180n
M1322 t478 t476 vdd vdd pch w=2u l=180n
CT481 t481 0 0.1f
M1323 t478 nw94 t481 0 nch w=1u l=180n
M1324 t481 t476 0 0 nch w=1u l=180n
M1325 nw182 t477 vdd vdd pch w=2u l=180n
M1326 nw182 t478 vdd vdd pch w=2u l=180n
CT482 t482 0 0.1f
M1327 nw182 t477 t482 0 nch w=1u l=180n
M1328 t482 t478 0 0 nch w=1u l=180n
Cnw182 nw182 0 2f
M1329 nw183 ni1 vdd vdd pch w=2u l=180n
M1330 nw183 nw96 vdd vdd pch w=2u l=180n
CT483 t483 0 0.1f
M1331 nw183 ni1 t483 0 nch w=1u l=180n
M1332 t483 nw96 0 0 nch w=1u l=180n
Cnw183 nw183 0 2f
M1333 nw184 ni2 0 0 nch w=1u l=180n
M1334 nw184 nw98 0 0 nch w=1u l=180n
CT484 t484 0 0.1f
M1335 t484 ni2 vdd vdd pch w=2u l=180n
M1336 nw184 nw98 t484 vdd pch w=2u l=180n
Cnw184 nw184 0 2f
CT485 t485 0 0.1f
M1337 t485 ni3 vdd vdd pch w=2u l=180n
M1338 t485 nw100 vdd vdd pch w=2u l=180n
CT486 t486 0 0.1f
M1339 t485 ni3 t486 0 nch w=1u l=180n
M1340 t486 nw100 0 0 nch w=1u l=180n
M1341 nw185 t485 vdd vdd pch w=2u l=180n
M1342 nw185 t485 0 0 nch w=1u l=180n
Cnw185 nw185 0 2f
CT487 t487 0 0.1f
M1343 t487 ni4 0 0 nch w=1u l=180n
M1344 t487 nw102 0 0 nch w=1u l=180n
CT488 t488 0 0.1f
M1345 t488 ni4 vdd vdd pch w=2u l=180n
M1346 t487 nw102 t488 vdd pch w=2u l=180n
M1347 nw186 t487 vdd vdd pch w=2u l=180n
M1348 nw186 t487 0 0 nch w=1u l=180n
Cnw186 nw186 0 2f
CT489 t489 0 0.1f
CT490 t490 0 0.1f
CT491 t491 0 0.1f
M1349 t489 ni5 vdd vdd pch w=2u l=180n
M1350 t489 nw104 vdd vdd pch w=2u l=180n
CT492 t492 0 0.1f
M1351 t489 ni5 t492 0 nch w=1u l=180n
M1352 t492 nw104 0 0 nch w=1u l=180n
M1353 t490 ni5 vdd vdd pch w=2u l=180n
M1354 t490 t489 vdd vdd pch w=2u l=180n
CT493 t493 0 0.1f
M1355 t490 ni5 t493 0 nch w=1u l=180n
M1356 t493 t489 0 0 nch w=1u l=180n
M1357 t491 nw104 vdd vdd pch w=2u l=180n
M1358 t491 t489 vdd vdd pch w=2u l=180n
CT494 t494 0 0.1f
M1359 t491 nw104 t494 0 nch w=1u l=180n
M1360 t494 t489 0 0 nch w=1u l=180n
M1361 nw187 t490 vdd vdd pch w=2u l=180n
M1362 nw187 t491 vdd vdd pch w=2u l=180n
CT495 t495 0 0.1f
M1363 nw187 t490 t495 0 nch w=1u l=180n
M1364 t495 t491 0 0 nch w=1u l=180n
Cnw187 nw187 0 2f
M1365 nw188 ni6 vdd vdd pch w=2u l=180n
M1366 nw188 nw106 vdd vdd pch w=2u l=180n
CT496 t496 0 0.1f
M1367 nw188 ni6 t496 0 nch w=1u l=180n
M1368 t496 nw106 0 0 nch w=1u l=180n
Cnw188 nw188 0 2f
M1369 nw189 ni7 0 0 nch w=1u l=180n
M1370 nw189 nw108 0 0 nch w=1u l=180n
CT497 t497 0 0.1f
M1371 t497 ni7 vdd vdd pch w=2u l=180n
M1372 nw189 nw108 t497 vdd pch w=2u l=180n
Cnw189 nw189 0 2f
CT498 t498 0 0.1f
M1373 t498 ni8 vdd vdd pch w=2u l=180n
M1374 t498 nw110 vdd vdd pch w=2u l=180n
CT499 t499 0 0.1f
M1375 t498 ni8 t499 0 nch w=1u l=180n
M1376 t499 nw110 0 0 nch w=1u l=180n
M1377 nw190 t498 vdd vdd pch w=2u l=180n
M1378 nw190 t498 0 0 nch w=1u l=180n
Cnw190 nw190 0 2f
CT500 t500 0 0.1f
M1379 t500 nw3 0 0 nch w=1u l=180n
M1380 t500 nw112 0 0 nch w=1u l=180n
CT501 t501 0 0.1f
M1381 t501 nw3 vdd vdd pch w=2u l=180n
M1382 t500 nw112 t501 vdd pch w=2u l=180n
M1383 nw191 t500 vdd vdd pch w=2u l=180n
M1384 nw191 t500 0 0 nch w=1u l=180n
Cnw191 nw191 0 2f
CT502 t502 0 0.1f
CT503 t503 0 0.1f
CT504 t504 0 0.1f
M1385 t502 nw4 vdd vdd pch w=2u l=180n
M1386 t502 nw114 vdd vdd pch w=2u l=180n
CT505 t505 0 0.1f
M1387 t502 nw4 t505 0 nch w=1u l=180n
M1388 t505 nw114 0 0 nch w=1u l=180n
M1389 t503 nw4 vdd vdd pch w=2u l=180n
M1390 t503 t502 vdd vdd pch w=2u l=180n
CT506 t506 0 0.1f
M1391 t503 nw4 t506 0 nch w=1u l=180n
M1392 t506 t502 0 0 nch w=1u l=180n
M1393 t504 nw114 vdd vdd pch w=2u l=180n
M1394 t504 t502 vdd vdd pch w=2u l=180n
CT507 t507 0 0.1f
M1395 t504 nw114 t507 0 nch w=1u l=180n
M1396 t507 t502 0 0 nch w=1u l=180n
M1397 nw192 t503 vdd vdd pch w=2u l=180n
M1398 nw192 t504 vdd vdd pch w=2u l=180n
CT508 t508 0 0.1f
M1399 nw192 t503 t508 0 nch w=1u l=180n
M1400 t508 t504 0 0 nch w=1u l=180n
Cnw192 nw192 0 2f
M1401 nw193 nw5 vdd vdd pch w=2u l=180n
M1402 nw193 nw116 vdd vdd pch w=2u l=180n
CT509 t509 0 0.1f
M1403 nw193 nw5 t509 0 nch w=1u l=180n
M1404 t509 nw116 0 0 nch w=1u l=180n
Cnw193 nw193 0 2f
M1405 nw194 nw6 0 0 nch w=1u l=180n
M1406 nw194 nw118 0 0 nch w=1u l=180n
CT510 t510 0 0.1f
M1407 t510 nw6 vdd vdd pch w=2u l=180n
M1408 nw194 nw118 t510 vdd pch w=2u l=180n
Cnw194 nw194 0 2f
CT511 t511 0 0.1f
M1409 t511 nw7 vdd vdd pch w=2u l=180n
M1410 t511 nw120 vdd vdd pch w=2u l=180n
CT512 t512 0 0.1f
M1411 t511 nw7 t512 0 nch w=1u l=180n
M1412 t512 nw120 0 0 nch w=1u l=180n
M1413 nw195 t511 vdd vdd pch w=2u l=180n
M1414 nw195 t511 0 0 nch w=1u l=180n
Cnw195 nw195 0 2f
CT513 t513 0 0.1f
M1415 t513 nw8 0 0 nch w=1u l=180n
M1416 t513 nw122 0 0 nch w=1u l=180n
CT514 t514 0 0.1f
M1417 t514 nw8 vdd vdd pch w=2u l=180n
M1418 t513 nw122 t514 vdd pch w=2u l=180n
M1419 nw196 t513 vdd vdd pch w=2u l=180n
M1420 nw196 t513 0 0 nch w=1u l=180n
Cnw196 nw196 0 2f
CT515 t515 0 0.1f
CT516 t516 0 0.1f
CT517 t517 0 0.1f
M1421 t515 nw9 vdd vdd pch w=2u l=180n
M1422 t515 nw124 vdd vdd pch w=2u l=180n
CT518 t518 0 0.1f
M1423 t515 nw9 t518 0 nch w=1u l=180n
M1424 t518 nw124 0 0 nch w=1u l=180n
M1425 t516 nw9 vdd vdd pch w=2u l=180n
M1426 t516 t515 vdd vdd pch w=2u l=180n
CT519 t519 0 0.1f
M1427 t516 nw9 t519 0 nch w=1u l=180n
M1428 t519 t515 0 0 nch w=1u l=180n
M1429 t517 nw124 vdd vdd pch w=2u l=180n
M1430 t517 t515 vdd vdd pch w=2u l=180n
CT520 t520 0 0.1f
M1431 t517 nw124 t520 0 nch w=1u l=180n
M1432 t520 t515 0 0 nch w=1u l=180n
M1433 nw197 t516 vdd vdd pch w=2u l=180n
M1434 nw197 t517 vdd vdd pch w=2u l=180n
CT521 t521 0 0.1f
M1435 nw197 t516 t521 0 nch w=1u l=180n
M1436 t521 t517 0 0 nch w=1u l=180n
Cnw197 nw197 0 2f
M1437 nw198 nw10 vdd vdd pch w=2u l=180n
M1438 nw198 nw126 vdd vdd pch w=2u l=180n
CT522 t522 0 0.1f
M1439 nw198 nw10 t522 0 nch w=1u l=180n
M1440 t522 nw126 0 0 nch w=1u l=180n
Cnw198 nw198 0 2f
M1441 nw199 nw11 0 0 nch w=1u l=180n
M1442 nw199 nw128 0 0 nch w=1u l=180n
CT523 t523 0 0.1f
M1443 t523 nw11 vdd vdd pch w=2u l=180n
M1444 nw199 nw128 t523 vdd pch w=2u l=180n
Cnw199 nw199 0 2f
CT524 t524 0 0.1f
M1445 t524 nw12 vdd vdd pch w=2u l=180n
M1446 t524 nw130 vdd vdd pch w=2u l=180n
CT525 t525 0 0.1f
M1447 t524 nw12 t525 0 nch w=1u l=180n
M1448 t525 nw130 0 0 nch w=1u l=180n
M1449 nw200 t524 vdd vdd pch w=2u l=180n
M1450 nw200 t524 0 0 nch w=1u l=180n
Cnw200 nw200 0 2f
CT526 t526 0 0.1f
M1451 t526 nw13 0 0 nch w=1u l=180n
M1452 t526 nw132 0 0 nch w=1u l=180n
CT527 t527 0 0.1f
M1453 t527 nw13 vdd vdd pch w=2u l=180n
M1454 t526 nw132 t527 vdd pch w=2u l=180n
M1455 nw201 t526 vdd vdd pch w=2u l=180n
M1456 nw201 t526 0 0 nch w=1u l=180n
Cnw201 nw201 0 2f
CT528 t528 0 0.1f
CT529 t529 0 0.1f
CT530 t530 0 0.1f
M1457 t528 nw14 vdd vdd pch w=2u l=180n
M1458 t528 nw134 vdd vdd pch w=2u l=180n
CT531 t531 0 0.1f
M1459 t528 nw14 t531 0 nch w=1u l=180n
M1460 t531 nw134 0 0 nch w=1u l=180n
M1461 t529 nw14 vdd vdd pch w=2u l=180n
M1462 t529 t528 vdd vdd pch w=2u l=180n
CT532 t532 0 0.1f
M1463 t529 nw14 t532 0 nch w=1u l=180n
M1464 t532 t528 0 0 nch w=1u l=180n
M1465 t530 nw134 vdd vdd pch w=2u l=180n
M1466 t530 t528 vdd vdd pch w=2u l=180n
CT533 t533 0 0.1f
M1467 t530 nw134 t533 0 nch w=1u l=180n
M1468 t533 t528 0 0 nch w=1u l=180n
M1469 nw202 t529 vdd vdd pch w=2u l=180n
M1470 nw202 t530 vdd vdd pch w=2u l=180n
CT534 t534 0 0.1f
M1471 nw202 t529 t534 0 nch w=1u l=180n
M1472 t534 t530 0 0 nch w=1u l=180n
Cnw202 nw202 0 2f
M1473 nw203 nw15 vdd vdd pch w=2u l=180n
M1474 nw203 nw136 vdd vdd pch w=2u l=180n
CT535 t535 0 0.1f
M1475 nw203 nw15 t535 0 nch w=1u l=180n
M1476 t535 nw136 0 0 nch w=1u l=180n
Cnw203 nw203 0 2f
M1477 nw204 nw16 0 0 nch w=1u l=180n
M1478 nw204 nw138 0 0 nch w=1u l=180n
CT536 t536 0 0.1f
M1479 t536 nw16 vdd vdd pch w=2u l=180n
M1480 nw204 nw138 t536 vdd pch w=2u l=180n
Cnw204 nw204 0 2f
CT537 t537 0 0.1f
M1481 t537 nw17 vdd vdd pch w=2u l=180n
M1482 t537 nw140 vdd vdd pch w=2u l=180n
CT538 t538 0 0.1f
M1483 t537 nw17 t538 0 nch w=1u l=180n
M1484 t538 nw140 0 0 nch w=1u l=180n
M1485 nw205 t537 vdd vdd pch w=2u l=180n
M1486 nw205 t537 0 0 nch w=1u l=180n
Cnw205 nw205 0 2f
CT539 t539 0 0.1f
M1487 t539 nw18 0 0 nch w=1u l=180n
M1488 t539 nw142 0 0 nch w=1u l=180n
CT540 t540 0 0.1f
M1489 t540 nw18 vdd vdd pch w=2u l=180n
M1490 t539 nw142 t540 vdd pch w=2u l=180n
M1491 nw206 t539 vdd vdd pch w=2u l=180n
M1492 nw206 t539 0 0 nch w=1u l=180n
Cnw206 nw206 0 2f
CT541 t541 0 0.1f
CT542 t542 0 0.1f
CT543 t543 0 0.1f
M1493 t541 nw19 vdd vdd pch w=2u l=180n
M1494 t541 nw144 vdd vdd pch w=2u l=180n
CT544 t544 0 0.1f
M1495 t541 nw19 t544 0 nch w=1u l=180n
M1496 t544 nw144 0 0 nch w=1u l=180n
M1497 t542 nw19 vdd vdd pch w=2u l=180n
M1498 t542 t541 vdd vdd pch w=2u l=180n
CT545 t545 0 0.1f
M1499 t542 nw19 t545 0 nch w=1u l=180n
M1500 t545 t541 0 0 nch w=1u l=180n
M1501 t543 nw144 vdd vdd pch w=2u l=180n
M1502 t543 t541 vdd vdd pch w=2u l=180n
CT546 t546 0 0.1f
M1503 t543 nw144 t546 0 nch w=1u l=180n
M1504 t546 t541 0 0 nch w=1u l=180n
M1505 nw207 t542 vdd vdd pch w=2u l=180n
M1506 nw207 t543 vdd vdd pch w=2u l=180n
CT547 t547 0 0.1f
M1507 nw207 t542 t547 0 nch w=1u l=180n
M1508 t547 t543 0 0 nch w=1u l=180n
Cnw207 nw207 0 2f
M1509 nw208 nw20 vdd vdd pch w=2u l=180n
M1510 nw208 nw146 vdd vdd pch w=2u l=180n
CT548 t548 0 0.1f
M1511 nw208 nw20 t548 0 nch w=1u l=180n
M1512 t548 nw146 0 0 nch w=1u l=180n
Cnw208 nw208 0 2f
M1513 nw209 nw21 0 0 nch w=1u l=180n
M1514 nw209 nw148 0 0 nch w=1u l=180n
CT549 t549 0 0.1f
M1515 t549 nw21 vdd vdd pch w=2u l=180n
M1516 nw209 nw148 t549 vdd pch w=2u l=180n
Cnw209 nw209 0 2f
CT550 t550 0 0.1f
M1517 t550 nw22 vdd vdd pch w=2u l=180n
M1518 t550 nw150 vdd vdd pch w=2u l=180n
CT551 t551 0 0.1f
M1519 t550 nw22 t551 0 nch w=1u l=180n
M1520 t551 nw150 0 0 nch w=1u l=180n
M1521 nw210 t550 vdd vdd pch w=2u l=180n
M1522 nw210 t550 0 0 nch w=1u l=180n
Cnw210 nw210 0 2f
CT552 t552 0 0.1f
M1523 t552 nw23 0 0 nch w=1u l=180n
M1524 t552 nw152 0 0 nch w=1u l=180n
CT553 t553 0 0.1f
M1525 t553 nw23 vdd vdd pch w=2u l=180n
M1526 t552 nw152 t553 vdd pch w=2u l=180n
M1527 nw211 t552 vdd vdd pch w=2u l=180n
M1528 nw211 t552 0 0 nch w=1u l=180n
Cnw211 nw211 0 2f
CT554 t554 0 0.1f
CT555 t555 0 0.1f
CT556 t556 0 0.1f
M1529 t554 nw24 vdd vdd pch w=2u l=180n
M1530 t554 nw154 vdd vdd pch w=2u l=180n
CT557 t557 0 0.1f
M1531 t554 nw24 t557 0 nch w=1u l=180n
M1532 t557 nw154 0 0 nch w=1u l=180n
M1533 t555 nw24 vdd vdd pch w=2u l=180n
M1534 t555 t554 vdd vdd pch w=2u l=180n
CT558 t558 0 0.1f
M1535 t555 nw24 t558 0 nch w=1u l=180n
M1536 t558 t554 0 0 nch w=1u l=180n
M1537 t556 nw154 vdd vdd pch w=2u l=180n
M1538 t556 t554 vdd vdd pch w=2u l=180n
CT559 t559 0 0.1f
M1539 t556 nw154 t559 0 nch w=1u l=180n
M1540 t559 t554 0 0 nch w=1u l=180n
M1541 nw212 t555 vdd vdd pch w=2u l=180n
M1542 nw212 t556 vdd vdd pch w=2u l=180n
CT560 t560 0 0.1f
M1543 nw212 t555 t560 0 nch w=1u l=180n
M1544 t560 t556 0 0 nch w=1u l=180n
Cnw212 nw212 0 2f
M1545 nw213 nw25 vdd vdd pch w=2u l=180n
M1546 nw213 nw156 vdd vdd pch w=2u l=180n
CT561 t561 0 0.1f
M1547 nw213 nw25 t561 0 nch w=1u l=180n
M1548 t561 nw156 0 0 nch w=1u l=180n
Cnw213 nw213 0 2f
M1549 nw214 nw26 0 0 nch w=1u l=180n
M1550 nw214 nw158 0 0 nch w=1u l=180n
CT562 t562 0 0.1f
M1551 t562 nw26 vdd vdd pch w=2u l=180n
M1552 nw214 nw158 t562 vdd pch w=2u l=180n
Cnw214 nw214 0 2f
CT563 t563 0 0.1f
M1553 t563 nw27 vdd vdd pch w=2u l=180n
M1554 t563 nw160 vdd vdd pch w=2u l=180n
CT564 t564 0 0.1f
M1555 t563 nw27 t564 0 nch w=1u l=180n
M1556 t564 nw160 0 0 nch w=1u l=180n
M1557 nw215 t563 vdd vdd pch w=2u l=180n
M1558 nw215 t563 0 0 nch w=1u l=180n
Cnw215 nw215 0 2f
CT565 t565 0 0.1f
M1559 t565 nw28 0 0 nch w=1u l=180n
M1560 t565 nw162 0 0 nch w=1u l=180n
CT566 t566 0 0.1f
M1561 t566 nw28 vdd vdd pch w=2u l=180n
M1562 t565 nw162 t566 vdd pch w=2u l=180n
M1563 nw216 t565 vdd vdd pch w=2u l=180n
M1564 nw216 t565 0 0 nch w=1u l=180n
Cnw216 nw216 0 2f
CT567 t567 0 0.1f
CT568 t568 0 0.1f
CT569 t569 0 0.1f
M1565 t567 nw29 vdd vdd pch w=2u l=180n
M1566 t567 nw164 vdd vdd pch w=2u l=180n
CT570 t570 0 0.1f
M1567 t567 nw29 t570 0 nch w=1u l=180n
M1568 t570 nw164 0 0 nch w=1u l=180n
M1569 t568 nw29 vdd vdd pch w=2u l=180n
M1570 t568 t567 vdd vdd pch w=2u l=180n
CT571 t571 0 0.1f
M1571 t568 nw29 t571 0 nch w=1u l=180n
M1572 t571 t567 0 0 nch w=1u l=180n
M1573 t569 nw164 vdd vdd pch w=2u l=180n
M1574 t569 t567 vdd vdd pch w=2u l=180n
CT572 t572 0 0.1f
M1575 t569 nw164 t572 0 nch w=1u l=180n
M1576 t572 t567 0 0 nch w=1u l=180n
M1577 nw217 t568 vdd vdd pch w=2u l=180n
M1578 nw217 t569 vdd vdd pch w=2u l=180n
CT573 t573 0 0.1f
M1579 nw217 t568 t573 0 nch w=1u l=180n
M1580 t573 t569 0 0 nch w=1u l=180n
Cnw217 nw217 0 2f
M1581 nw218 nw30 vdd vdd pch w=2u l=180n
M1582 nw218 nw166 vdd vdd pch w=2u l=180n
CT574 t574 0 0.1f
M1583 nw218 nw30 t574 0 nch w=1u l=180n
M1584 t574 nw166 0 0 nch w=1u l=180n
Cnw218 nw218 0 2f
M1585 nw219 nw31 0 0 nch w=1u l=180n
M1586 nw219 nw168 0 0 nch w=1u l=180n
CT575 t575 0 0.1f
M1587 t575 nw31 vdd vdd pch w=2u l=180n
M1588 nw219 nw168 t575 vdd pch w=2u l=180n
Cnw219 nw219 0 2f
CT576 t576 0 0.1f
M1589 t576 nw32 vdd vdd pch w=2u l=180n
M1590 t576 nw170 vdd vdd pch w=2u l=180n
CT577 t577 0 0.1f
M1591 t576 nw32 t577 0 nch w=1u l=180n
M1592 t577 nw170 0 0 nch w=1u l=180n
M1593 nw220 t576 vdd vdd pch w=2u l=180n
M1594 nw220 t576 0 0 nch w=1u l=180n
Cnw220 nw220 0 2f
CT578 t578 0 0.1f
M1595 t578 nw33 0 0 nch w=1u l=180n
M1596 t578 nw172 0 0 nch w=1u l=180n
CT579 t579 0 0.1f
M1597 t579 nw33 vdd vdd pch w=2u l=180n
M1598 t578 nw172 t579 vdd pch w=2u l=180n
M1599 nw221 t578 vdd vdd pch w=2u l=180n
M1600 nw221 t578 0 0 nch w=1u l=180n
Cnw221 nw221 0 2f
CT580 t580 0 0.1f
CT581 t581 0 0.1f
CT582 t582 0 0.1f
M1601 t580 nw34 vdd vdd pch w=2u l=180n
M1602 t580 nw174 vdd vdd pch w=2u l=180n
CT583 t583 0 0.1f
M1603 t580 nw34 t583 0 nch w=1u l=180n
M1604 t583 nw174 0 0 nch w=1u l=180n
M1605 t581 nw34 vdd vdd pch w=2u l=180n
M1606 t581 t580 vdd vdd pch w=2u l=180n
CT584 t584 0 0.1f
M1607 t581 nw34 t584 0 nch w=1u l=180n
M1608 t584 t580 0 0 nch w=1u l=180n
M1609 t582 nw174 vdd vdd pch w=2u l=180n
M1610 t582 t580 vdd vdd pch w=2u l=180n
CT585 t585 0 0.1f
M1611 t582 nw174 t585 0 nch w=1u l=180n
M1612 t585 t580 0 0 nch w=1u l=180n
M1613 nw222 t581 vdd vdd pch w=2u l=180n
M1614 nw222 t582 vdd vdd pch w=2u l=180n
CT586 t586 0 0.1f
M1615 nw222 t581 t586 0 nch w=1u l=180n
M1616 t586 t582 0 0 nch w=1u l=180n
Cnw222 nw222 0 2f
M1617 nw223 nw35 vdd vdd pch w=2u l=180n
M1618 nw223 nw176 vdd vdd pch w=2u l=180n
CT587 t587 0 0.1f
M1619 nw223 nw35 t587 0 nch w=1u l=180n
M1620 t587 nw176 0 0 nch w=1u l=180n
Cnw223 nw223 0 2f
M1621 nw224 nw36 0 0 nch w=1u l=180n
M1622 nw224 nw178 0 0 nch w=1u l=180n
CT588 t588 0 0.1f
M1623 t588 nw36 vdd vdd pch w=2u l=180n
M1624 nw224 nw178 t588 vdd pch w=2u l=180n
Cnw224 nw224 0 2f
CT589 t589 0 0.1f
M1625 t589 nw37 vdd vdd pch w=2u l=180n
M1626 t589 nw180 vdd vdd pch w=2u l=180n
CT590 t590 0 0.1f
M1627 t589 nw37 t590 0 nch w=1u l=180n
M1628 t590 nw180 0 0 nch w=1u l=180n
M1629 nw225 t589 vdd vdd pch w=2u l=180n
M1630 nw225 t589 0 0 nch w=1u l=180n
Cnw225 nw225 0 2f
CT591 t591 0 0.1f
M1631 t591 nw38 0 0 nch w=1u l=180n
M1632 t591 nw182 0 0 nch w=1u l=180n
CT592 t592 0 0.1f
M1633 t592 nw38 vdd vdd pch w=2u l=180n
M1634 t591 nw182 t592 vdd pch w=2u l=180n
M1635 nw226 t591 vdd vdd pch w=2u l=180n
M1636 nw226 t591 0 0 nch w=1u l=180n
Cnw226 nw226 0 2f
CT593 t593 0 0.1f
CT594 t594 0 0.1f
CT595 t595 0 0.1f
M1637 t593 nw39 vdd vdd pch w=2u l=180n
M1638 t593 nw184 vdd vdd pch w=2u l=180n
CT596 t596 0 0.1f
M1639 t593 nw39 t596 0 nch w=1u l=180n
M1640 t596 nw184 0 0 nch w=1u l=180n
M1641 t594 nw39 vdd vdd pch w=2u l=180n
M1642 t594 t593 vdd vdd pch w=2u l=180n
CT597 t597 0 0.1f
M1643 t594 nw39 t597 0 nch w=1u l=180n
M1644 t597 t593 0 0 nch w=1u l=180n
M1645 t595 nw184 vdd vdd pch w=2u l=180n
M1646 t595 t593 vdd vdd pch w=2u l=180n
CT598 t598 0 0.1f
M1647 t595 nw184 t598 0 nch w=1u l=180n
M1648 t598 t593 0 0 nch w=1u l=180n
M1649 nw227 t594 vdd vdd pch w=2u l=180n
M1650 nw227 t595 vdd vdd pch w=2u l=180n
CT599 t599 0 0.1f
M1651 nw227 t594 t599 0 nch w=1u l=180n
M1652 t599 t595 0 0 nch w=1u l=180n
Cnw227 nw227 0 2f
M1653 nw228 nw40 vdd vdd pch w=2u l=180n
M1654 nw228 nw186 vdd vdd pch w=2u l=180n
CT600 t600 0 0.1f
M1655 nw228 nw40 t600 0 nch w=1u l=180n
M1656 t600 nw186 0 0 nch w=1u l=180n
Cnw228 nw228 0 2f
M1657 nw229 nw41 0 0 nch w=1u l=180n
M1658 nw229 nw188 0 0 nch w=1u l=180n
CT601 t601 0 0.1f
M1659 t601 nw41 vdd vdd pch w=2u l=180n
M1660 nw229 nw188 t601 vdd pch w=2u l=180n
Cnw229 nw229 0 2f
CT602 t602 0 0.1f
M1661 t602 nw42 vdd vdd pch w=2u l=180n
M1662 t602 nw190 vdd vdd pch w=2u l=180n
CT603 t603 0 0.1f
M1663 t602 nw42 t603 0 nch w=1u l=180n
M1664 t603 nw190 0 0 nch w=1u l=180n
M1665 nw230 t602 vdd vdd pch w=2u l=180n
M1666 nw230 t602 0 0 nch w=1u l=180n
Cnw230 nw230 0 2f
CT604 t604 0 0.1f
M1667 t604 nw43 0 0 nch w=1u l=180n
M1668 t604 nw192 0 0 nch w=1u l=180n
CT605 t605 0 0.1f
M1669 t605 nw43 vdd vdd pch w=2u l=180n
M1670 t604 nw192 t605 vdd pch w=2u l=180n
M1671 nw231 t604 vdd vdd pch w=2u l=180n
M1672 nw231 t604 0 0 nch w=1u l=180n
Cnw231 nw231 0 2f
CT606 t606 0 0.1f
CT607 t607 0 0.1f
CT608 t608 0 0.1f
M1673 t606 nw44 vdd vdd pch w=2u l=180n
M1674 t606 nw194 vdd vdd pch w=2u l=180n
CT609 t609 0 0.1f
M1675 t606 nw44 t609 0 nch w=1u l=180n
M1676 t609 nw194 0 0 nch w=1u l=180n
M1677 t607 nw44 vdd vdd pch w=2u l=180n
M1678 t607 t606 vdd vdd pch w=2u l=180n
CT610 t610 0 0.1f
M1679 t607 nw44 t610 0 nch w=1u l=180n
M1680 t610 t606 0 0 nch w=1u l=180n
M1681 t608 nw194 vdd vdd pch w=2u l=180n
M1682 t608 t606 vdd vdd pch w=2u l=180n
CT611 t611 0 0.1f
M1683 t608 nw194 t611 0 nch w=1u l=180n
M1684 t611 t606 0 0 nch w=1u l=180n
M1685 nw232 t607 vdd vdd pch w=2u l=180n
M1686 nw232 t608 vdd vdd pch w=2u l=180n
CT612 t612 0 0.1f
M1687 nw232 t607 t612 0 nch w=1u l=180n
M1688 t612 t608 0 0 nch w=1u l=180n
Cnw232 nw232 0 2f
M1689 nw233 nw45 vdd vdd pch w=2u l=180n
M1690 nw233 nw196 vdd vdd pch w=2u l=180n
CT613 t613 0 0.1f
M1691 nw233 nw45 t613 0 nch w=1u l=180n
M1692 t613 nw196 0 0 nch w=1u l=180n
Cnw233 nw233 0 2f
M1693 nw234 nw46 0 0 nch w=1u l=180n
M1694 nw234 nw198 0 0 nch w=1u l=180n
CT614 t614 0 0.1f
M1695 t614 nw46 vdd vdd pch w=2u l=180n
M1696 nw234 nw198 t614 vdd pch w=2u l=180n
Cnw234 nw234 0 2f
CT615 t615 0 0.1f
M1697 t615 nw47 vdd vdd pch w=2u l=180n
M1698 t615 nw200 vdd vdd pch w=2u l=180n
CT616 t616 0 0.1f
M1699 t615 nw47 t616 0 nch w=1u l=180n
M1700 t616 nw200 0 0 nch w=1u l=180n
M1701 nw235 t615 vdd vdd pch w=2u l=180n
M1702 nw235 t615 0 0 nch w=1u l=180n
Cnw235 nw235 0 2f
CT617 t617 0 0.1f
M1703 t617 nw48 0 0 nch w=1u l=180n
M1704 t617 nw202 0 0 nch w=1u l=180n
CT618 t618 0 0.1f
M1705 t618 nw48 vdd vdd pch w=2u l=180n
M1706 t617 nw202 t618 vdd pch w=2u l=180n
M1707 nw236 t617 vdd vdd pch w=2u l=180n
M1708 nw236 t617 0 0 nch w=1u l=180n
Cnw236 nw236 0 2f
CT619 t619 0 0.1f
CT620 t620 0 0.1f
CT621 t621 0 0.1f
M1709 t619 nw49 vdd vdd pch w=2u l=180n
M1710 t619 nw204 vdd vdd pch w=2u l=180n
CT622 t622 0 0.1f
M1711 t619 nw49 t622 0 nch w=1u l=180n
M1712 t622 nw204 0 0 nch w=1u l=180n
M1713 t620 nw49 vdd vdd pch w=2u l=180n
M1714 t620 t619 vdd vdd pch w=2u l=180n
CT623 t623 0 0.1f
M1715 t620 nw49 t623 0 nch w=1u l=180n
M1716 t623 t619 0 0 nch w=1u l=180n
M1717 t621 nw204 vdd vdd pch w=2u l=180n
M1718 t621 t619 vdd vdd pch w=2u l=180n
CT624 t624 0 0.1f
M1719 t621 nw204 t624 0 nch w=1u l=180n
M1720 t624 t619 0 0 nch w=1u l=180n
M1721 nw237 t620 vdd vdd pch w=2u l=180n
M1722 nw237 t621 vdd vdd pch w=2u l=180n
CT625 t625 0 0.1f
M1723 nw237 t620 t625 0 nch w=1u l=180n
M1724 t625 t621 0 0 nch w=1u l=180n
Cnw237 nw237 0 2f
M1725 nw238 nw50 vdd vdd pch w=2u l=180n
M1726 nw238 nw206 vdd vdd pch w=2u l=180n
CT626 t626 0 0.1f
M1727 nw238 nw50 t626 0 nch w=1u l=180n
M1728 t626 nw206 0 0 nch w=1u l=180n
Cnw238 nw238 0 2f
M1729 nw239 nw51 0 0 nch w=1u l=180n
M1730 nw239 nw208 0 0 nch w=1u l=180n
CT627 t627 0 0.1f
M1731 t627 nw51 vdd vdd pch w=2u l=180n
M1732 nw239 nw208 t627 vdd pch w=2u l=180n
Cnw239 nw239 0 2f
CT628 t628 0 0.1f
M1733 t628 nw52 vdd vdd pch w=2u l=180n
M1734 t628 nw210 vdd vdd pch w=2u l=180n
CT629 t629 0 0.1f
M1735 t628 nw52 t629 0 nch w=1u l=180n
M1736 t629 nw210 0 0 nch w=1u l=180n
M1737 nw240 t628 vdd vdd pch w=2u l=180n
M1738 nw240 t628 0 0 nch w=1u l=180n
Cnw240 nw240 0 2f
CT630 t630 0 0.1f
M1739 t630 nw53 0 0 nch w=1u l=180n
M1740 t630 nw212 0 0 nch w=1u l=180n
CT631 t631 0 0.1f
M1741 t631 nw53 vdd vdd pch w=2u l=180n
M1742 t630 nw212 t631 vdd pch w=2u l=180n
M1743 nw241 t630 vdd vdd pch w=2u l=180n
M1744 nw241 t630 0 0 nch w=1u l=180n
Cnw241 nw241 0 2f
CT632 t632 0 0.1f
CT633 t633 0 0.1f
CT634 t634 0 0.1f
M1745 t632 nw54 vdd vdd pch w=2u l=180n
M1746 t632 nw214 vdd vdd pch w=2u l=180n
CT635 t635 0 0.1f
M1747 t632 nw54 t635 0 nch w=1u l=180n
M1748 t635 nw214 0 0 nch w=1u l=180n
M1749 t633 nw54 vdd vdd pch w=2u l=180n
M1750 t633 t632 vdd vdd pch w=2u l=180n
CT636 t636 0 0.1f
M1751 t633 nw54 t636 0 nch w=1u l=180n
M1752 t636 t632 0 0 nch w=1u l=180n
M1753 t634 nw214 vdd vdd pch w=2u l=180n
M1754 t634 t632 vdd vdd pch w=2u l=180n
CT637 t637 0 0.1f
M1755 t634 nw214 t637 0 nch w=1u l=180n
M1756 t637 t632 0 0 nch w=1u l=180n
M1757 nw242 t633 vdd vdd pch w=2u l=180n
M1758 nw242 t634 vdd vdd pch w=2u l=180n
CT638 t638 0 0.1f
M1759 nw242 t633 t638 0 nch w=1u l=180n
M1760 t638 t634 0 0 nch w=1u l=180n
Cnw242 nw242 0 2f
M1761 nw243 nw55 vdd vdd pch w=2u l=180n
M1762 nw243 nw216 vdd vdd pch w=2u l=180n
CT639 t639 0 0.1f
M1763 nw243 nw55 t639 0 nch w=1u l=180n
M1764 t639 nw216 0 0 nch w=1u l=180n
Cnw243 nw243 0 2f
M1765 nw244 nw56 0 0 nch w=1u l=180n
M1766 nw244 nw218 0 0 nch w=1u l=180n
CT640 t640 0 0.1f
M1767 t640 nw56 vdd vdd pch w=2u l=180n
M1768 nw244 nw218 t640 vdd pch w=2u l=180n
Cnw244 nw244 0 2f
CT641 t641 0 0.1f
M1769 t641 nw57 vdd vdd pch w=2u l=180n
M1770 t641 nw220 vdd vdd pch w=2u l=180n
CT642 t642 0 0.1f
M1771 t641 nw57 t642 0 nch w=1u l=180n
M1772 t642 nw220 0 0 nch w=1u l=180n
M1773 nw245 t641 vdd vdd pch w=2u l=180n
M1774 nw245 t641 0 0 nch w=1u l=180n
Cnw245 nw245 0 2f
CT643 t643 0 0.1f
M1775 t643 nw58 0 0 nch w=1u l=180n
M1776 t643 nw222 0 0 nch w=1u l=180n
CT644 t644 0 0.1f
M1777 t644 nw58 vdd vdd pch w=2u l=180n
M1778 t643 nw222 t644 vdd pch w=2u l=180n
M1779 nw246 t643 vdd vdd pch w=2u l=180n
M1780 nw246 t643 0 0 nch w=1u l=180n
Cnw246 nw246 0 2f
CT645 t645 0 0.1f
CT646 t646 0 0.1f
CT647 t647 0 0.1f
M1781 t645 nw59 vdd vdd pch w=2u l=180n
M1782 t645 nw224 vdd vdd pch w=2u l=180n
CT648 t648 0 0.1f
M1783 t645 nw59 t648 0 nch w=1u l=180n
M1784 t648 nw224 0 0 nch w=1u l=180n
M1785 t646 nw59 vdd vdd pch w=2u l=180n
M1786 t646 t645 vdd vdd pch w=2u l=180n
CT649 t649 0 0.1f
M1787 t646 nw59 t649 0 nch w=1u l=180n
M1788 t649 t645 0 0 nch w=1u l=180n
M1789 t647 nw224 vdd vdd pch w=2u l=180n
M1790 t647 t645 vdd vdd pch w=2u l=180n
CT650 t650 0 0.1f
M1791 t647 nw224 t650 0 nch w=1u l=180n
M1792 t650 t645 0 0 nch w=1u l=180n
M1793 nw247 t646 vdd vdd pch w=2u l=180n
M1794 nw247 t647 vdd vdd pch w=2u l=180n
CT651 t651 0 0.1f
M1795 nw247 t646 t651 0 nch w=1u l=180n
M1796 t651 t647 0 0 nch w=1u l=180n
Cnw247 nw247 0 2f
M1797 nw248 nw60 vdd vdd pch w=2u l=180n
M1798 nw248 nw226 vdd vdd pch w=2u l=180n
CT652 t652 0 0.1f
M1799 nw248 nw60 t652 0 nch w=1u l=180n
M1800 t652 nw226 0 0 nch w=1u l=180n
Cnw248 nw248 0 2f
M1801 nw249 nw61 0 0 nch w=1u l=180n
M1802 nw249 nw228 0 0 nch w=1u l=180n
CT653 t653 0 0.1f
M1803 t653 nw61 vdd vdd pch w=2u l=180n
M1804 nw249 nw228 t653 vdd pch w=2u l=180n
Cnw249 nw249 0 2f
CT654 t654 0 0.1f
M1805 t654 nw62 vdd vdd pch w=2u l=180n
M1806 t654 nw230 vdd vdd pch w=2u l=180n
CT655 t655 0 0.1f
M1807 t654 nw62 t655 0 nch w=1u l=180n
M1808 t655 nw230 0 0 nch w=1u l=180n
M1809 nw250 t654 vdd vdd pch w=2u l=180n
M1810 nw250 t654 0 0 nch w=1u l=180n
Cnw250 nw250 0 2f
CT656 t656 0 0.1f
M1811 t656 nw63 0 0 nch w=1u l=180n
M1812 t656 nw232 0 0 nch w=1u l=180n
CT657 t657 0 0.1f
M1813 t657 nw63 vdd vdd pch w=2u l=180n
M1814 t656 nw232 t657 vdd pch w=2u l=180n
M1815 nw251 t656 vdd vdd pch w=2u l=180n
M1816 nw251 t656 0 0 nch w=1u l=180n
Cnw251 nw251 0 2f
CT658 t658 0 0.1f
CT659 t659 0 0.1f
CT660 t660 0 0.1f
M1817 t658 nw64 vdd vdd pch w=2u l=180n
M1818 t658 nw234 vdd vdd pch w=2u l=180n
CT661 t661 0 0.1f
M1819 t658 nw64 t661 0 nch w=1u l=180n
M1820 t661 nw234 0 0 nch w=1u l=180n
M1821 t659 nw64 vdd vdd pch w=2u l=180n
M1822 t659 t658 vdd vdd pch w=2u l=180n
CT662 t662 0 0.1f
M1823 t659 nw64 t662 0 nch w=1u l=180n
M1824 t662 t658 0 0 nch w=1u l=180n
M1825 t660 nw234 vdd vdd pch w=2u l=180n
M1826 t660 t658 vdd vdd pch w=2u l=180n
CT663 t663 0 0.1f
M1827 t660 nw234 t663 0 nch w=1u l=180n
M1828 t663 t658 0 0 nch w=1u l=180n
M1829 nw252 t659 vdd vdd pch w=2u l=180n
M1830 nw252 t660 vdd vdd pch w=2u l=180n
CT664 t664 0 0.1f
M1831 nw252 t659 t664 0 nch w=1u l=180n
M1832 t664 t660 0 0 nch w=1u l=180n
Cnw252 nw252 0 2f
M1833 nw253 nw65 vdd vdd pch w=2u l=180n
M1834 nw253 nw236 vdd vdd pch w=2u l=180n
CT665 t665 0 0.1f
M1835 nw253 nw65 t665 0 nch w=1u l=180n
M1836 t665 nw236 0 0 nch w=1u l=180n
Cnw253 nw253 0 2f
M1837 nw254 nw66 0 0 nch w=1u l=180n
M1838 nw254 nw238 0 0 nch w=1u l=180n
CT666 t666 0 0.1f
M1839 t666 nw66 vdd vdd pch w=2u l=180n
M1840 nw254 nw238 t666 vdd pch w=2u l=180n
Cnw254 nw254 0 2f
CT667 t667 0 0.1f
M1841 t667 nw67 vdd vdd pch w=2u l=180n
M1842 t667 nw240 vdd vdd pch w=2u l=180n
CT668 t668 0 0.1f
M1843 t667 nw67 t668 0 nch w=1u l=180n
M1844 t668 nw240 0 0 nch w=1u l=180n
M1845 nw255 t667 vdd vdd pch w=2u l=180n
M1846 nw255 t667 0 0 nch w=1u l=180n
Cnw255 nw255 0 2f
CT669 t669 0 0.1f
M1847 t669 nw68 0 0 nch w=1u l=180n
M1848 t669 nw242 0 0 nch w=1u l=180n
CT670 t670 0 0.1f
M1849 t670 nw68 vdd vdd pch w=2u l=180n
M1850 t669 nw242 t670 vdd pch w=2u l=180n
M1851 nw256 t669 vdd vdd pch w=2u l=180n
M1852 nw256 t669 0 0 nch w=1u l=180n
Cnw256 nw256 0 2f
CT671 t671 0 0.1f
CT672 t672 0 0.1f
CT673 t673 0 0.1f
M1853 t671 nw69 vdd vdd pch w=2u l=180n
M1854 t671 nw244 vdd vdd pch w=2u l=180n
CT674 t674 0 0.1f
M1855 t671 nw69 t674 0 nch w=1u l=180n
M1856 t674 nw244 0 0 nch w=1u l=180n
M1857 t672 nw69 vdd vdd pch w=2u l=180n
M1858 t672 t671 vdd vdd pch w=2u l=180n
CT675 t675 0 0.1f
M1859 t672 nw69 t675 0 nch w=1u l=180n
M1860 t675 t671 0 0 nch w=1u l=180n
M1861 t673 nw244 vdd vdd pch w=2u l=180n
M1862 t673 t671 vdd vdd pch w=2u l=180n
CT676 t676 0 0.1f
M1863 t673 nw244 t676 0 nch w=1u l=180n
M1864 t676 t671 0 0 nch w=1u l=180n
M1865 nw257 t672 vdd vdd pch w=2u l=180n
M1866 nw257 t673 vdd vdd pch w=2u l=180n
CT677 t677 0 0.1f
M1867 nw257 t672 t677 0 nch w=1u l=180n
M1868 t677 t673 0 0 nch w=1u l=180n
Cnw257 nw257 0 2f
M1869 nw258 nw70 vdd vdd pch w=2u l=180n
M1870 nw258 nw246 vdd vdd pch w=2u l=180n
CT678 t678 0 0.1f
M1871 nw258 nw70 t678 0 nch w=1u l=180n
M1872 t678 nw246 0 0 nch w=1u l=180n
Cnw258 nw258 0 2f
M1873 nw259 nw71 0 0 nch w=1u l=180n
M1874 nw259 nw248 0 0 nch w=1u l=180n
CT679 t679 0 0.1f
M1875 t679 nw71 vdd vdd pch w=2u l=180n
M1876 nw259 nw248 t679 vdd pch w=2u l=180n
Cnw259 nw259 0 2f
CT680 t680 0 0.1f
M1877 t680 nw72 vdd vdd pch w=2u l=180n
M1878 t680 nw250 vdd vdd pch w=2u l=180n
CT681 t681 0 0.1f
M1879 t680 nw72 t681 0 nch w=1u l=180n
M1880 t681 nw250 0 0 nch w=1u l=180n
M1881 nw260 t680 vdd vdd pch w=2u l=180n
M1882 nw260 t680 0 0 nch w=1u l=180n
Cnw260 nw260 0 2f
CT682 t682 0 0.1f
M1883 t682 nw73 0 0 nch w=1u l=180n
M1884 t682 nw252 0 0 nch w=1u l=180n
CT683 t683 0 0.1f
M1885 t683 nw73 vdd vdd pch w=2u l=180n
M1886 t682 nw252 t683 vdd pch w=2u l=180n
M1887 nw261 t682 vdd vdd pch w=2u l=180n
M1888 nw261 t682 0 0 nch w=1u l=180n
Cnw261 nw261 0 2f
CT684 t684 0 0.1f
CT685 t685 0 0.1f
CT686 t686 0 0.1f
M1889 t684 nw74 vdd vdd pch w=2u l=180n
M1890 t684 nw254 vdd vdd pch w=2u l=180n
CT687 t687 0 0.1f
M1891 t684 nw74 t687 0 nch w=1u l=180n
M1892 t687 nw254 0 0 nch w=1u l=180n
M1893 t685 nw74 vdd vdd pch w=2u l=180n
M1894 t685 t684 vdd vdd pch w=2u l=180n
CT688 t688 0 0.1f
M1895 t685 nw74 t688 0 nch w=1u l=180n
M1896 t688 t684 0 0 nch w=1u l=180n
M1897 t686 nw254 vdd vdd pch w=2u l=180n
M1898 t686 t684 vdd vdd pch w=2u l=180n
CT689 t689 0 0.1f
M1899 t686 nw254 t689 0 nch w=1u l=180n
M1900 t689 t684 0 0 nch w=1u l=180n
M1901 nw262 t685 vdd vdd pch w=2u l=180n
M1902 nw262 t686 vdd vdd pch w=2u l=180n
CT690 t690 0 0.1f
M1903 nw262 t685 t690 0 nch w=1u l=180n
M1904 t690 t686 0 0 nch w=1u l=180n
Cnw262 nw262 0 2f
M1905 nw263 nw75 vdd vdd pch w=2u l=180n
M1906 nw263 nw256 vdd vdd pch w=2u l=180n
CT691 t691 0 0.1f
M1907 nw263 nw75 t691 0 nch w=1u l=180n
M1908 t691 nw256 0 0 nch w=1u l=180n
Cnw263 nw263 0 2f
M1909 nw264 nw76 0 0 nch w=1u l=180n
M1910 nw264 nw258 0 0 nch w=1u l=180n
CT692 t692 0 0.1f
M1911 t692 nw76 vdd vdd pch w=2u l=180n
M1912 nw264 nw258 t692 vdd pch w=2u l=180n
Cnw264 nw264 0 2f
CT693 t693 0 0.1f
M1913 t693 nw77 vdd vdd pch w=2u l=180n
M1914 t693 nw260 vdd vdd pch w=2u l=180n
CT694 t694 0 0.1f
M1915 t693 nw77 t694 0 nch w=1u l=180n
M1916 t694 nw260 0 0 nch w=1u l=180n
M1917 nw265 t693 vdd vdd pch w=2u l=180n
M1918 nw265 t693 0 0 nch w=1u l=180n
Cnw265 nw265 0 2f
CT695 t695 0 0.1f
M1919 t695 nw78 0 0 nch w=1u l=180n
M1920 t695 nw262 0 0 nch w=1u l=180n
CT696 t696 0 0.1f
M1921 t696 nw78 vdd vdd pch w=2u l=180n
M1922 t695 nw262 t696 vdd pch w=2u l=180n
M1923 nw266 t695 vdd vdd pch w=2u l=180n
M1924 nw266 t695 0 0 nch w=1u l=180n
Cnw266 nw266 0 2f
CT697 t697 0 0.1f
CT698 t698 0 0.1f
CT699 t699 0 0.1f
M1925 t697 nw79 vdd vdd pch w=2u l=180n
M1926 t697 nw264 vdd vdd pch w=2u l=180n
CT700 t700 0 0.1f
M1927 t697 nw79 t700 0 nch w=1u l=180n
M1928 t700 nw264 0 0 nch w=1u l=180n
M1929 t698 nw79 vdd vdd pch w=2u l=180n
M1930 t698 t697 vdd vdd pch w=2u l=180n
CT701 t701 0 0.1f
M1931 t698 nw79 t701 0 nch w=1u l=180n
M1932 t701 t697 0 0 nch w=1u l=180n
M1933 t699 nw264 vdd vdd pch w=2u l=180n
M1934 t699 t697 vdd vdd pch w=2u l=180n
CT702 t702 0 0.1f
M1935 t699 nw264 t702 0 nch w=1u l=180n
M1936 t702 t697 0 0 nch w=1u l=180n
M1937 nw267 t698 vdd vdd pch w=2u l=180n
M1938 nw267 t699 vdd vdd pch w=2u l=180n
CT703 t703 0 0.1f
M1939 nw267 t698 t703 0 nch w=1u l=180n
M1940 t703 t699 0 0 nch w=1u l=180n
Cnw267 nw267 0 2f
M1941 nw268 nw80 vdd vdd pch w=2u l=180n
M1942 nw268 nw266 vdd vdd pch w=2u l=180n
CT704 t704 0 0.1f
M1943 nw268 nw80 t704 0 nch w=1u l=180n
M1944 t704 nw266 0 0 nch w=1u l=180n
Cnw268 nw268 0 2f
M1945 nw269 nw81 0 0 nch w=1u l=180n
M1946 nw269 nw268 0 0 nch w=1u l=180n
CT705 t705 0 0.1f
M1947 t705 nw81 vdd vdd pch w=2u l=180n
M1948 nw269 nw268 t705 vdd pch w=2u l=180n
Cnw269 nw269 0 2f
CT706 t706 0 0.1f
M1949 t706 nw82 vdd vdd pch w=2u l=180n
M1950 t706 nq0 vdd vdd pch w=2u l=180n
CT707 t707 0 0.1f
M1951 t706 nw82 t707 0 nch w=1u l=180n
M1952 t707 nq0 0 0 nch w=1u l=180n
M1953 nw270 t706 vdd vdd pch w=2u l=180n
M1954 nw270 t706 0 0 nch w=1u l=180n
Cnw270 nw270 0 2f
CT708 t708 0 0.1f
M1955 t708 nw83 0 0 nch w=1u l=180n
M1956 t708 nq1 0 0 nch w=1u l=180n
CT709 t709 0 0.1f
M1957 t709 nw83 vdd vdd pch w=2u l=180n
M1958 t708 nq1 t709 vdd pch w=2u l=180n
M1959 nw271 t708 vdd vdd pch w=2u l=180n
M1960 nw271 t708 0 0 nch w=1u l=180n
Cnw271 nw271 0 2f
CT710 t710 0 0.1f
CT711 t711 0 0.1f
CT712 t712 0 0.1f
M1961 t710 nw84 vdd vdd pch w=2u l=180n
M1962 t710 nq2 vdd vdd pch w=2u l=180n
CT713 t713 0 0.1f
M1963 t710 nw84 t713 0 nch w=1u l=180n
M1964 t713 nq2 0 0 nch w=1u l=180n
M1965 t711 nw84 vdd vdd pch w=2u l=180n
M1966 t711 t710 vdd vdd pch w=2u l=180n
CT714 t714 0 0.1f
M1967 t711 nw84 t714 0 nch w=1u l=180n
M1968 t714 t710 0 0 nch w=1u l=180n
M1969 t712 nq2 vdd vdd pch w=2u l=180n
M1970 t712 t710 vdd vdd pch w=2u l=180n
CT715 t715 0 0.1f
M1971 t712 nq2 t715 0 nch w=1u l=180n
M1972 t715 t710 0 0 nch w=1u l=180n
M1973 nw272 t711 vdd vdd pch w=2u l=180n
M1974 nw272 t712 vdd vdd pch w=2u l=180n
CT716 t716 0 0.1f
M1975 nw272 t711 t716 0 nch w=1u l=180n
M1976 t716 t712 0 0 nch w=1u l=180n
Cnw272 nw272 0 2f
M1977 nw273 nw85 vdd vdd pch w=2u l=180n
M1978 nw273 nq3 vdd vdd pch w=2u l=180n
CT717 t717 0 0.1f
M1979 nw273 nw85 t717 0 nch w=1u l=180n
M1980 t717 nq3 0 0 nch w=1u l=180n
Cnw273 nw273 0 2f
M1981 nw274 nw86 0 0 nch w=1u l=180n
M1982 nw274 nq4 0 0 nch w=1u l=180n
CT718 t718 0 0.1f
M1983 t718 nw86 vdd vdd pch w=2u l=180n
M1984 nw274 nq4 t718 vdd pch w=2u l=180n
Cnw274 nw274 0 2f
CT719 t719 0 0.1f
M1985 t719 nw87 vdd vdd pch w=2u l=180n
M1986 t719 nq5 vdd vdd pch w=2u l=180n
CT720 t720 0 0.1f
M1987 t719 nw87 t720 0 nch w=1u l=180n
M1988 t720 nq5 0 0 nch w=1u l=180n
M1989 nw275 t719 vdd vdd pch w=2u l=180n
M1990 nw275 t719 0 0 nch w=1u l=180n
Cnw275 nw275 0 2f
CT721 t721 0 0.1f
M1991 t721 nw88 0 0 nch w=1u l=180n
M1992 t721 nq6 0 0 nch w=1u l=180n
CT722 t722 0 0.1f
M1993 t722 nw88 vdd vdd pch w=2u l=180n
M1994 t721 nq6 t722 vdd pch w=2u l=180n
M1995 nw276 t721 vdd vdd pch w=2u l=180n
M1996 nw276 t721 0 0 nch w=1u l=180n
Cnw276 nw276 0 2f
CT723 t723 0 0.1f
CT724 t724 0 0.1f
CT725 t725 0 0.1f
M1997 t723 nw89 vdd vdd pch w=2u l=180n
M1998 t723 nq7 vdd vdd pch w=2u l=180n
CT726 t726 0 0.1f
M1999 t723 nw89 t726 0 nch w=1u l=180n
M2000 t726 nq7 0 0 nch w=1u l=180n
M2001 t724 nw89 vdd vdd pch w=2u l=180n
M2002 t724 t723 vdd vdd pch w=2u l=180n
CT727 t727 0 0.1f
M2003 t724 nw89 t727 0 nch w=1u l=180n
M2004 t727 t723 0 0 nch w=1u l=180n
M2005 t725 nq7 vdd vdd pch w=2u l=180n
M2006 t725 t723 vdd vdd pch w=2u l=180n
CT728 t728 0 0.1f
M2007 t725 nq7 t728 0 nch w=1u l=180n
M2008 t728 t723 0 0 nch w=1u l=180n
M2009 nw277 t724 vdd vdd pch w=2u l=180n
M2010 nw277 t725 vdd vdd pch w=2u l=180n
CT729 t729 0 0.1f
M2011 nw277 t724 t729 0 nch w=1u l=180n
M2012 t729 t725 0 0 nch w=1u l=180n
Cnw277 nw277 0 2f
M2013 nw278 nw90 vdd vdd pch w=2u l=180n
M2014 nw278 nq8 vdd vdd pch w=2u l=180n
CT730 t730 0 0.1f
M2015 nw278 nw90 t730 0 nch w=1u l=180n
M2016 t730 nq8 0 0 nch w=1u l=180n
Cnw278 nw278 0 2f
M2017 nw279 nw91 0 0 nch w=1u l=180n
M2018 nw279 nq9 0 0 nch w=1u l=180n
CT731 t731 0 0.1f
M2019 t731 nw91 vdd vdd pch w=2u l=180n
M2020 nw279 nq9 t731 vdd pch w=2u l=180n
Cnw279 nw279 0 2f
CT732 t732 0 0.1f
M2021 t732 nw92 vdd vdd pch w=2u l=180n
M2022 t732 nq10 vdd vdd pch w=2u l=180n
CT733 t733 0 0.1f
M2023 t732 nw92 t733 0 nch w=1u l=180n
M2024 t733 nq10 0 0 nch w=1u l=180n
M2025 nw280 t732 vdd vdd pch w=2u l=180n
M2026 nw280 t732 0 0 nch w=1u l=180n
Cnw280 nw280 0 2f
CT734 t734 0 0.1f
M2027 t734 nw93 0 0 nch w=1u l=180n
M2028 t734 nq11 0 0 nch w=1u l=180n
CT735 t735 0 0.1f
M2029 t735 nw93 vdd vdd pch w=2u l=180n
M2030 t734 nq11 t735 vdd pch w=2u l=180n
M2031 nw281 t734 vdd vdd pch w=2u l=180n
M2032 nw281 t734 0 0 nch w=1u l=180n
Cnw281 nw281 0 2f
CT736 t736 0 0.1f
CT737 t737 0 0.1f
CT738 t738 0 0.1f
M2033 t736 nw94 vdd vdd pch w=2u l=180n
M2034 t736 nq12 vdd vdd pch w=2u l=180n
CT739 t739 0 0.1f
M2035 t736 nw94 t739 0 nch w=1u l=180n
M2036 t739 nq12 0 0 nch w=1u l=180n
M2037 t737 nw94 vdd vdd pch w=2u l=180n
M2038 t737 t736 vdd vdd pch w=2u l=180n
CT740 t740 0 0.1f
M2039 t737 nw94 t740 0 nch w=1u l=180n
M2040 t740 t736 0 0 nch w=1u l=180n
M2041 t738 nq12 vdd vdd pch w=2u l=180n
M2042 t738 t736 vdd vdd pch w=2u l=180n
CT741 t741 0 0.1f
M2043 t738 nq12 t741 0 nch w=1u l=180n
M2044 t741 t736 0 0 nch w=1u l=180n
M2045 nw282 t737 vdd vdd pch w=2u l=180n
M2046 nw282 t738 vdd vdd pch w=2u l=180n
CT742 t742 0 0.1f
M2047 nw282 t737 t742 0 nch w=1u l=180n
M2048 t742 t738 0 0 nch w=1u l=180n
Cnw282 nw282 0 2f
M2049 nw283 nw95 vdd vdd pch w=2u l=180n
M2050 nw283 nq13 vdd vdd pch w=2u l=180n
CT743 t743 0 0.1f
M2051 nw283 nw95 t743 0 nch w=1u l=180n
M2052 t743 nq13 0 0 nch w=1u l=180n
Cnw283 nw283 0 2f
M2053 nw284 nw96 0 0 nch w=1u l=180n
M2054 nw284 nq14 0 0 nch w=1u l=180n
CT744 t744 0 0.1f
M2055 t744 nw96 vdd vdd pch w=2u l=180n
M2056 nw284 nq14 t744 vdd pch w=2u l=180n
Cnw284 nw284 0 2f
CT745 t745 0 0.1f
M2057 t745 nw97 vdd vdd pch w=2u l=180n
M2058 t745 nq15 vdd vdd pch w=2u l=180n
CT746 t746 0 0.1f
M2059 t745 nw97 t746 0 nch w=1u l=180n
M2060 t746 nq15 0 0 nch w=1u l=180n
M2061 nw285 t745 vdd vdd pch w=2u l=180n
M2062 nw285 t745 0 0 nch w=1u l=180n
Cnw285 nw285 0 2f
CT747 t747 0 0.1f
M2063 t747 nw98 0 0 nch w=1u l=180n
M2064 t747 nq16 0 0 nch w=1u l=180n
CT748 t748 0 0.1f
M2065 t748 nw98 vdd vdd pch w=2u l=180n
M2066 t747 nq16 t748 vdd pch w=2u l=180n
M2067 nw286 t747 vdd vdd pch w=2u l=180n
M2068 nw286 t747 0 0 nch w=1u l=180n
Cnw286 nw286 0 2f
CT749 t749 0 0.1f
CT750 t750 0 0.1f
CT751 t751 0 0.1f
M2069 t749 nw99 vdd vdd pch w=2u l=180n
M2070 t749 nq17 vdd vdd pch w=2u l=180n
CT752 t752 0 0.1f
M2071 t749 nw99 t752 0 nch w=1u l=180n
M2072 t752 nq17 0 0 nch w=1u l=180n
M2073 t750 nw99 vdd vdd pch w=2u l=180n
M2074 t750 t749 vdd vdd pch w=2u l=180n
CT753 t753 0 0.1f
M2075 t750 nw99 t753 0 nch w=1u l=180n
M2076 t753 t749 0 0 nch w=1u l=180n
M2077 t751 nq17 vdd vdd pch w=2u l=180n
M2078 t751 t749 vdd vdd pch w=2u l=180n
CT754 t754 0 0.1f
M2079 t751 nq17 t754 0 nch w=1u l=180n
M2080 t754 t749 0 0 nch w=1u l=180n
M2081 nw287 t750 vdd vdd pch w=2u l=180n
M2082 nw287 t751 vdd vdd pch w=2u l=180n
CT755 t755 0 0.1f
M2083 nw287 t750 t755 0 nch w=1u l=180n
M2084 t755 t751 0 0 nch w=1u l=180n
Cnw287 nw287 0 2f
M2085 nw288 nw100 vdd vdd pch w=2u l=180n
M2086 nw288 ni0 vdd vdd pch w=2u l=180n
CT756 t756 0 0.1f
M2087 nw288 nw100 t756 0 nch w=1u l=180n
M2088 t756 ni0 0 0 nch w=1u l=180n
Cnw288 nw288 0 2f
M2089 nw289 nw101 0 0 nch w=1u l=180n
M2090 nw289 ni1 0 0 nch w=1u l=180n
CT757 t757 0 0.1f
M2091 t757 nw101 vdd vdd pch w=2u l=180n
M2092 nw289 ni1 t757 vdd pch w=2u l=180n
Cnw289 nw289 0 2f
CT758 t758 0 0.1f
M2093 t758 nw102 vdd vdd pch w=2u l=180n
M2094 t758 ni2 vdd vdd pch w=2u l=180n
CT759 t759 0 0.1f
M2095 t758 nw102 t759 0 nch w=1u l=180n
M2096 t759 ni2 0 0 nch w=1u l=180n
M2097 nw290 t758 vdd vdd pch w=2u l=180n
M2098 nw290 t758 0 0 nch w=1u l=180n
Cnw290 nw290 0 2f
CT760 t760 0 0.1f
M2099 t760 nw103 0 0 nch w=1u l=180n
M2100 t760 ni3 0 0 nch w=1u l=180n
CT761 t761 0 0.1f
M2101 t761 nw103 vdd vdd pch w=2u l=180n
M2102 t760 ni3 t761 vdd pch w=2u l=180n
M2103 nw291 t760 vdd vdd pch w=2u l=180n
M2104 nw291 t760 0 0 nch w=1u l=180n
Cnw291 nw291 0 2f
CT762 t762 0 0.1f
CT763 t763 0 0.1f
CT764 t764 0 0.1f
M2105 t762 nw104 vdd vdd pch w=2u l=180n
M2106 t762 ni4 vdd vdd pch w=2u l=180n
CT765 t765 0 0.1f
M2107 t762 nw104 t765 0 nch w=1u l=180n
M2108 t765 ni4 0 0 nch w=1u l=180n
M2109 t763 nw104 vdd vdd pch w=2u l=180n
M2110 t763 t762 vdd vdd pch w=2u l=180n
CT766 t766 0 0.1f
M2111 t763 nw104 t766 0 nch w=1u l=180n
M2112 t766 t762 0 0 nch w=1u l=180n
M2113 t764 ni4 vdd vdd pch w=2u l=180n
M2114 t764 t762 vdd vdd pch w=2u l=180n
CT767 t767 0 0.1f
M2115 t764 ni4 t767 0 nch w=1u l=180n
M2116 t767 t762 0 0 nch w=1u l=180n
M2117 nw292 t763 vdd vdd pch w=2u l=180n
M2118 nw292 t764 vdd vdd pch w=2u l=180n
CT768 t768 0 0.1f
M2119 nw292 t763 t768 0 nch w=1u l=180n
M2120 t768 t764 0 0 nch w=1u l=180n
Cnw292 nw292 0 2f
M2121 nw293 nw105 vdd vdd pch w=2u l=180n
M2122 nw293 ni5 vdd vdd pch w=2u l=180n
CT769 t769 0 0.1f
M2123 nw293 nw105 t769 0 nch w=1u l=180n
M2124 t769 ni5 0 0 nch w=1u l=180n
Cnw293 nw293 0 2f
M2125 nw294 nw106 0 0 nch w=1u l=180n
M2126 nw294 ni6 0 0 nch w=1u l=180n
CT770 t770 0 0.1f
M2127 t770 nw106 vdd vdd pch w=2u l=180n
M2128 nw294 ni6 t770 vdd pch w=2u l=180n
Cnw294 nw294 0 2f
CT771 t771 0 0.1f
M2129 t771 nw107 vdd vdd pch w=2u l=180n
M2130 t771 ni7 vdd vdd pch w=2u l=180n
CT772 t772 0 0.1f
M2131 t771 nw107 t772 0 nch w=1u l=180n
M2132 t772 ni7 0 0 nch w=1u l=180n
M2133 nw295 t771 vdd vdd pch w=2u l=180n
M2134 nw295 t771 0 0 nch w=1u l=180n
Cnw295 nw295 0 2f
CT773 t773 0 0.1f
M2135 t773 nw108 0 0 nch w=1u l=180n
M2136 t773 ni8 0 0 nch w=1u l=180n
CT774 t774 0 0.1f
M2137 t774 nw108 vdd vdd pch w=2u l=180n
M2138 t773 ni8 t774 vdd pch w=2u l=180n
M2139 nw296 t773 vdd vdd pch w=2u l=180n
M2140 nw296 t773 0 0 nch w=1u l=180n
Cnw296 nw296 0 2f
CT775 t775 0 0.1f
CT776 t776 0 0.1f
CT777 t777 0 0.1f
M2141 t775 nw109 vdd vdd pch w=2u l=180n
M2142 t775 nw3 vdd vdd pch w=2u l=180n
CT778 t778 0 0.1f
M2143 t775 nw109 t778 0 nch w=1u l=180n
M2144 t778 nw3 0 0 nch w=1u l=180n
M2145 t776 nw109 vdd vdd pch w=2u l=180n
M2146 t776 t775 vdd vdd pch w=2u l=180n
CT779 t779 0 0.1f
M2147 t776 nw109 t779 0 nch w=1u l=180n
M2148 t779 t775 0 0 nch w=1u l=180n
M2149 t777 nw3 vdd vdd pch w=2u l=180n
M2150 t777 t775 vdd vdd pch w=2u l=180n
CT780 t780 0 0.1f
M2151 t777 nw3 t780 0 nch w=1u l=180n
M2152 t780 t775 0 0 nch w=1u l=180n
M2153 nw297 t776 vdd vdd pch w=2u l=180n
M2154 nw297 t777 vdd vdd pch w=2u l=180n
CT781 t781 0 0.1f
M2155 nw297 t776 t781 0 nch w=1u l=180n
M2156 t781 t777 0 0 nch w=1u l=180n
Cnw297 nw297 0 2f
M2157 nw298 nw110 vdd vdd pch w=2u l=180n
M2158 nw298 nw4 vdd vdd pch w=2u l=180n
CT782 t782 0 0.1f
M2159 nw298 nw110 t782 0 nch w=1u l=180n
M2160 t782 nw4 0 0 nch w=1u l=180n
Cnw298 nw298 0 2f
M2161 nw299 nw111 0 0 nch w=1u l=180n
M2162 nw299 nw5 0 0 nch w=1u l=180n
CT783 t783 0 0.1f
M2163 t783 nw111 vdd vdd pch w=2u l=180n
M2164 nw299 nw5 t783 vdd pch w=2u l=180n
Cnw299 nw299 0 2f
CT784 t784 0 0.1f
M2165 t784 nw112 vdd vdd pch w=2u l=180n
M2166 t784 nw6 vdd vdd pch w=2u l=180n
CT785 t785 0 0.1f
M2167 t784 nw112 t785 0 nch w=1u l=180n
M2168 t785 nw6 0 0 nch w=1u l=180n
M2169 nw300 t784 vdd vdd pch w=2u l=180n
M2170 nw300 t784 0 0 nch w=1u l=180n
Cnw300 nw300 0 2f
CT786 t786 0 0.1f
M2171 t786 nw113 0 0 nch w=1u l=180n
M2172 t786 nw7 0 0 nch w=1u l=180n
CT787 t787 0 0.1f
M2173 t787 nw113 vdd vdd pch w=2u l=180n
M2174 t786 nw7 t787 vdd pch w=2u l=180n
M2175 nw301 t786 vdd vdd pch w=2u l=180n
M2176 nw301 t786 0 0 nch w=1u l=180n
Cnw301 nw301 0 2f
CT788 t788 0 0.1f
CT789 t789 0 0.1f
CT790 t790 0 0.1f
M2177 t788 nw114 vdd vdd pch w=2u l=180n
M2178 t788 nw8 vdd vdd pch w=2u l=180n
CT791 t791 0 0.1f
M2179 t788 nw114 t791 0 nch w=1u l=180n
M2180 t791 nw8 0 0 nch w=1u l=180n
M2181 t789 nw114 vdd vdd pch w=2u l=180n
M2182 t789 t788 vdd vdd pch w=2u l=180n
CT792 t792 0 0.1f
M2183 t789 nw114 t792 0 nch w=1u l=180n
M2184 t792 t788 0 0 nch w=1u l=180n
M2185 t790 nw8 vdd vdd pch w=2u l=180n
M2186 t790 t788 vdd vdd pch w=2u l=180n
CT793 t793 0 0.1f
M2187 t790 nw8 t793 0 nch w=1u l=180n
M2188 t793 t788 0 0 nch w=1u l=180n
M2189 nw302 t789 vdd vdd pch w=2u l=180n
M2190 nw302 t790 vdd vdd pch w=2u l=180n
CT794 t794 0 0.1f
M2191 nw302 t789 t794 0 nch w=1u l=180n
M2192 t794 t790 0 0 nch w=1u l=180n
Cnw302 nw302 0 2f
M2193 nw303 nw115 vdd vdd pch w=2u l=180n
M2194 nw303 nw9 vdd vdd pch w=2u l=180n
CT795 t795 0 0.1f
M2195 nw303 nw115 t795 0 nch w=1u l=180n
M2196 t795 nw9 0 0 nch w=1u l=180n
Cnw303 nw303 0 2f
M2197 nw304 nw116 0 0 nch w=1u l=180n
M2198 nw304 nw10 0 0 nch w=1u l=180n
CT796 t796 0 0.1f
M2199 t796 nw116 vdd vdd pch w=2u l=180n
M2200 nw304 nw10 t796 vdd pch w=2u l=180n
Cnw304 nw304 0 2f
CT797 t797 0 0.1f
M2201 t797 nw117 vdd vdd pch w=2u l=180n
M2202 t797 nw11 vdd vdd pch w=2u l=180n
CT798 t798 0 0.1f
M2203 t797 nw117 t798 0 nch w=1u l=180n
M2204 t798 nw11 0 0 nch w=1u l=180n
M2205 nw305 t797 vdd vdd pch w=2u l=180n
M2206 nw305 t797 0 0 nch w=1u l=180n
Cnw305 nw305 0 2f
CT799 t799 0 0.1f
M2207 t799 nw118 0 0 nch w=1u l=180n
M2208 t799 nw12 0 0 nch w=1u l=180n
CT800 t800 0 0.1f
M2209 t800 nw118 vdd vdd pch w=2u l=180n
M2210 t799 nw12 t800 vdd pch w=2u l=180n
M2211 nw306 t799 vdd vdd pch w=2u l=180n
M2212 nw306 t799 0 0 nch w=1u l=180n
Cnw306 nw306 0 2f
CT801 t801 0 0.1f
CT802 t802 0 0.1f
CT803 t803 0 0.1f
M2213 t801 nw119 vdd vdd pch w=2u l=180n
M2214 t801 nw13 vdd vdd pch w=2u l=180n
CT804 t804 0 0.1f
M2215 t801 nw119 t804 0 nch w=1u l=180n
M2216 t804 nw13 0 0 nch w=1u l=180n
M2217 t802 nw119 vdd vdd pch w=2u l=180n
M2218 t802 t801 vdd vdd pch w=2u l=180n
CT805 t805 0 0.1f
M2219 t802 nw119 t805 0 nch w=1u l=180n
M2220 t805 t801 0 0 nch w=1u l=180n
M2221 t803 nw13 vdd vdd pch w=2u l=180n
M2222 t803 t801 vdd vdd pch w=2u l=180n
CT806 t806 0 0.1f
M2223 t803 nw13 t806 0 nch w=1u l=180n
M2224 t806 t801 0 0 nch w=1u l=180n
M2225 nw307 t802 vdd vdd pch w=2u l=180n
M2226 nw307 t803 vdd vdd pch w=2u l=180n
CT807 t807 0 0.1f
M2227 nw307 t802 t807 0 nch w=1u l=180n
M2228 t807 t803 0 0 nch w=1u l=180n
Cnw307 nw307 0 2f
M2229 nw308 nw120 vdd vdd pch w=2u l=180n
M2230 nw308 nw14 vdd vdd pch w=2u l=180n
CT808 t808 0 0.1f
M2231 nw308 nw120 t808 0 nch w=1u l=180n
M2232 t808 nw14 0 0 nch w=1u l=180n
Cnw308 nw308 0 2f
M2233 nw309 nw121 0 0 nch w=1u l=180n
M2234 nw309 nw15 0 0 nch w=1u l=180n
CT809 t809 0 0.1f
M2235 t809 nw121 vdd vdd pch w=2u l=180n
M2236 nw309 nw15 t809 vdd pch w=2u l=180n
Cnw309 nw309 0 2f
CT810 t810 0 0.1f
M2237 t810 nw122 vdd vdd pch w=2u l=180n
M2238 t810 nw16 vdd vdd pch w=2u l=180n
CT811 t811 0 0.1f
M2239 t810 nw122 t811 0 nch w=1u l=180n
M2240 t811 nw16 0 0 nch w=1u l=180n
M2241 nw310 t810 vdd vdd pch w=2u l=180n
M2242 nw310 t810 0 0 nch w=1u l=180n
Cnw310 nw310 0 2f
CT812 t812 0 0.1f
M2243 t812 nw123 0 0 nch w=1u l=180n
M2244 t812 nw17 0 0 nch w=1u l=180n
CT813 t813 0 0.1f
M2245 t813 nw123 vdd vdd pch w=2u l=180n
M2246 t812 nw17 t813 vdd pch w=2u l=180n
M2247 nw311 t812 vdd vdd pch w=2u l=180n
M2248 nw311 t812 0 0 nch w=1u l=180n
Cnw311 nw311 0 2f
CT814 t814 0 0.1f
CT815 t815 0 0.1f
CT816 t816 0 0.1f
M2249 t814 nw124 vdd vdd pch w=2u l=180n
M2250 t814 nw18 vdd vdd pch w=2u l=180n
CT817 t817 0 0.1f
M2251 t814 nw124 t817 0 nch w=1u l=180n
M2252 t817 nw18 0 0 nch w=1u l=180n
M2253 t815 nw124 vdd vdd pch w=2u l=180n
M2254 t815 t814 vdd vdd pch w=2u l=180n
CT818 t818 0 0.1f
M2255 t815 nw124 t818 0 nch w=1u l=180n
M2256 t818 t814 0 0 nch w=1u l=180n
M2257 t816 nw18 vdd vdd pch w=2u l=180n
M2258 t816 t814 vdd vdd pch w=2u l=180n
CT819 t819 0 0.1f
M2259 t816 nw18 t819 0 nch w=1u l=180n
M2260 t819 t814 0 0 nch w=1u l=180n
M2261 nw312 t815 vdd vdd pch w=2u l=180n
M2262 nw312 t816 vdd vdd pch w=2u l=180n
CT820 t820 0 0.1f
M2263 nw312 t815 t820 0 nch w=1u l=180n
M2264 t820 t816 0 0 nch w=1u l=180n
Cnw312 nw312 0 2f
M2265 nw313 nw125 vdd vdd pch w=2u l=180n
M2266 nw313 nw19 vdd vdd pch w=2u l=180n
CT821 t821 0 0.1f
M2267 nw313 nw125 t821 0 nch w=1u l=180n
M2268 t821 nw19 0 0 nch w=1u l=180n
Cnw313 nw313 0 2f
M2269 nw314 nw126 0 0 nch w=1u l=180n
M2270 nw314 nw20 0 0 nch w=1u l=180n
CT822 t822 0 0.1f
M2271 t822 nw126 vdd vdd pch w=2u l=180n
M2272 nw314 nw20 t822 vdd pch w=2u l=180n
Cnw314 nw314 0 2f
CT823 t823 0 0.1f
M2273 t823 nw127 vdd vdd pch w=2u l=180n
M2274 t823 nw21 vdd vdd pch w=2u l=180n
CT824 t824 0 0.1f
M2275 t823 nw127 t824 0 nch w=1u l=180n
M2276 t824 nw21 0 0 nch w=1u l=180n
M2277 nw315 t823 vdd vdd pch w=2u l=180n
M2278 nw315 t823 0 0 nch w=1u l=180n
Cnw315 nw315 0 2f
CT825 t825 0 0.1f
M2279 t825 nw128 0 0 nch w=1u l=180n
M2280 t825 nw22 0 0 nch w=1u l=180n
CT826 t826 0 0.1f
M2281 t826 nw128 vdd vdd pch w=2u l=180n
M2282 t825 nw22 t826 vdd pch w=2u l=180n
M2283 nw316 t825 vdd vdd pch w=2u l=180n
M2284 nw316 t825 0 0 nch w=1u l=180n
Cnw316 nw316 0 2f
CT827 t827 0 0.1f
CT828 t828 0 0.1f
CT829 t829 0 0.1f
M2285 t827 nw129 vdd vdd pch w=2u l=180n
M2286 t827 nw23 vdd vdd pch w=2u l=180n
CT830 t830 0 0.1f
M2287 t827 nw129 t830 0 nch w=1u l=180n
M2288 t830 nw23 0 0 nch w=1u l=180n
M2289 t828 nw129 vdd vdd pch w=2u l=180n
M2290 t828 t827 vdd vdd pch w=2u l=180n
CT831 t831 0 0.1f
M2291 t828 nw129 t831 0 nch w=1u l=180n
M2292 t831 t827 0 0 nch w=1u l=180n
M2293 t829 nw23 vdd vdd pch w=2u l=180n
M2294 t829 t827 vdd vdd pch w=2u l=180n
CT832 t832 0 0.1f
M2295 t829 nw23 t832 0 nch w=1u l=180n
M2296 t832 t827 0 0 nch w=1u l=180n
M2297 nw317 t828 vdd vdd pch w=2u l=180n
M2298 nw317 t829 vdd vdd pch w=2u l=180n
CT833 t833 0 0.1f
M2299 nw317 t828 t833 0 nch w=1u l=180n
M2300 t833 t829 0 0 nch w=1u l=180n
Cnw317 nw317 0 2f
M2301 nw318 nw130 vdd vdd pch w=2u l=180n
M2302 nw318 nw24 vdd vdd pch w=2u l=180n
CT834 t834 0 0.1f
M2303 nw318 nw130 t834 0 nch w=1u l=180n
M2304 t834 nw24 0 0 nch w=1u l=180n
Cnw318 nw318 0 2f
M2305 nw319 nw131 0 0 nch w=1u l=180n
M2306 nw319 nw25 0 0 nch w=1u l=180n
CT835 t835 0 0.1f
M2307 t835 nw131 vdd vdd pch w=2u l=180n
M2308 nw319 nw25 t835 vdd pch w=2u l=180n
Cnw319 nw319 0 2f
CT836 t836 0 0.1f
M2309 t836 nw132 vdd vdd pch w=2u l=180n
M2310 t836 nw26 vdd vdd pch w=2u l=180n
CT837 t837 0 0.1f
M2311 t836 nw132 t837 0 nch w=1u l=180n
M2312 t837 nw26 0 0 nch w=1u l=180n
M2313 nw320 t836 vdd vdd pch w=2u l=180n
M2314 nw320 t836 0 0 nch w=1u l=180n
Cnw320 nw320 0 2f
CT838 t838 0 0.1f
M2315 t838 nw133 0 0 nch w=1u l=180n
M2316 t838 nw27 0 0 nch w=1u l=180n
CT839 t839 0 0.1f
M2317 t839 nw133 vdd vdd pch w=2u l=180n
M2318 t838 nw27 t839 vdd pch w=2u l=180n
M2319 nw321 t838 vdd vdd pch w=2u l=180n
M2320 nw321 t838 0 0 nch w=1u l=180n
Cnw321 nw321 0 2f
CT840 t840 0 0.1f
CT841 t841 0 0.1f
CT842 t842 0 0.1f
M2321 t840 nw134 vdd vdd pch w=2u l=180n
M2322 t840 nw28 vdd vdd pch w=2u l=180n
CT843 t843 0 0.1f
M2323 t840 nw134 t843 0 nch w=1u l=180n
M2324 t843 nw28 0 0 nch w=1u l=180n
M2325 t841 nw134 vdd vdd pch w=2u l=180n
M2326 t841 t840 vdd vdd pch w=2u l=180n
CT844 t844 0 0.1f
M2327 t841 nw134 t844 0 nch w=1u l=180n
M2328 t844 t840 0 0 nch w=1u l=180n
M2329 t842 nw28 vdd vdd pch w=2u l=180n
M2330 t842 t840 vdd vdd pch w=2u l=180n
CT845 t845 0 0.1f
M2331 t842 nw28 t845 0 nch w=1u l=180n
M2332 t845 t840 0 0 nch w=1u l=180n
M2333 nw322 t841 vdd vdd pch w=2u l=180n
M2334 nw322 t842 vdd vdd pch w=2u l=180n
CT846 t846 0 0.1f
M2335 nw322 t841 t846 0 nch w=1u l=180n
M2336 t846 t842 0 0 nch w=1u l=180n
Cnw322 nw322 0 2f
M2337 nw323 nw135 vdd vdd pch w=2u l=180n
M2338 nw323 nw29 vdd vdd pch w=2u l=180n
CT847 t847 0 0.1f
M2339 nw323 nw135 t847 0 nch w=1u l=180n
M2340 t847 nw29 0 0 nch w=1u l=180n
Cnw323 nw323 0 2f
M2341 nw324 nw136 0 0 nch w=1u l=180n
M2342 nw324 nw30 0 0 nch w=1u l=180n
CT848 t848 0 0.1f
M2343 t848 nw136 vdd vdd pch w=2u l=180n
M2344 nw324 nw30 t848 vdd pch w=2u l=180n
Cnw324 nw324 0 2f
CT849 t849 0 0.1f
M2345 t849 nw137 vdd vdd pch w=2u l=180n
M2346 t849 nw31 vdd vdd pch w=2u l=180n
CT850 t850 0 0.1f
M2347 t849 nw137 t850 0 nch w=1u l=180n
M2348 t850 nw31 0 0 nch w=1u l=180n
M2349 nw325 t849 vdd vdd pch w=2u l=180n
M2350 nw325 t849 0 0 nch w=1u l=180n
Cnw325 nw325 0 2f
CT851 t851 0 0.1f
M2351 t851 nw138 0 0 nch w=1u l=180n
M2352 t851 nw32 0 0 nch w=1u l=180n
CT852 t852 0 0.1f
M2353 t852 nw138 vdd vdd pch w=2u l=180n
M2354 t851 nw32 t852 vdd pch w=2u l=180n
M2355 nw326 t851 vdd vdd pch w=2u l=180n
M2356 nw326 t851 0 0 nch w=1u l=180n
Cnw326 nw326 0 2f
CT853 t853 0 0.1f
CT854 t854 0 0.1f
CT855 t855 0 0.1f
M2357 t853 nw139 vdd vdd pch w=2u l=180n
M2358 t853 nw33 vdd vdd pch w=2u l=180n
CT856 t856 0 0.1f
M2359 t853 nw139 t856 0 nch w=1u l=180n
M2360 t856 nw33 0 0 nch w=1u l=180n
M2361 t854 nw139 vdd vdd pch w=2u l=180n
M2362 t854 t853 vdd vdd pch w=2u l=180n
CT857 t857 0 0.1f
M2363 t854 nw139 t857 0 nch w=1u l=180n
M2364 t857 t853 0 0 nch w=1u l=180n
M2365 t855 nw33 vdd vdd pch w=2u l=180n
M2366 t855 t853 vdd vdd pch w=2u l=180n
CT858 t858 0 0.1f
M2367 t855 nw33 t858 0 nch w=1u l=180n
M2368 t858 t853 0 0 nch w=1u l=180n
M2369 nw327 t854 vdd vdd pch w=2u l=180n
M2370 nw327 t855 vdd vdd pch w=2u l=180n
CT859 t859 0 0.1f
M2371 nw327 t854 t859 0 nch w=1u l=180n
M2372 t859 t855 0 0 nch w=1u l=180n
Cnw327 nw327 0 2f
M2373 nw328 nw140 vdd vdd pch w=2u l=180n
M2374 nw328 nw34 vdd vdd pch w=2u l=180n
CT860 t860 0 0.1f
M2375 nw328 nw140 t860 0 nch w=1u l=180n
M2376 t860 nw34 0 0 nch w=1u l=180n
Cnw328 nw328 0 2f
M2377 nw329 nw141 0 0 nch w=1u l=180n
M2378 nw329 nw35 0 0 nch w=1u l=180n
CT861 t861 0 0.1f
M2379 t861 nw141 vdd vdd pch w=2u l=180n
M2380 nw329 nw35 t861 vdd pch w=2u l=180n
Cnw329 nw329 0 2f
CT862 t862 0 0.1f
M2381 t862 nw142 vdd vdd pch w=2u l=180n
M2382 t862 nw36 vdd vdd pch w=2u l=180n
CT863 t863 0 0.1f
M2383 t862 nw142 t863 0 nch w=1u l=180n
M2384 t863 nw36 0 0 nch w=1u l=180n
M2385 nw330 t862 vdd vdd pch w=2u l=180n
M2386 nw330 t862 0 0 nch w=1u l=180n
Cnw330 nw330 0 2f
CT864 t864 0 0.1f
M2387 t864 nw143 0 0 nch w=1u l=180n
M2388 t864 nw37 0 0 nch w=1u l=180n
CT865 t865 0 0.1f
M2389 t865 nw143 vdd vdd pch w=2u l=180n
M2390 t864 nw37 t865 vdd pch w=2u l=180n
M2391 nw331 t864 vdd vdd pch w=2u l=180n
M2392 nw331 t864 0 0 nch w=1u l=180n
Cnw331 nw331 0 2f
CT866 t866 0 0.1f
CT867 t867 0 0.1f
CT868 t868 0 0.1f
M2393 t866 nw144 vdd vdd pch w=2u l=180n
M2394 t866 nw38 vdd vdd pch w=2u l=180n
CT869 t869 0 0.1f
M2395 t866 nw144 t869 0 nch w=1u l=180n
M2396 t869 nw38 0 0 nch w=1u l=180n
M2397 t867 nw144 vdd vdd pch w=2u l=180n
M2398 t867 t866 vdd vdd pch w=2u l=180n
CT870 t870 0 0.1f
M2399 t867 nw144 t870 0 nch w=1u l=180n
M2400 t870 t866 0 0 nch w=1u l=180n
M2401 t868 nw38 vdd vdd pch w=2u l=180n
M2402 t868 t866 vdd vdd pch w=2u l=180n
CT871 t871 0 0.1f
M2403 t868 nw38 t871 0 nch w=1u l=180n
M2404 t871 t866 0 0 nch w=1u l=180n
M2405 nw332 t867 vdd vdd pch w=2u l=180n
M2406 nw332 t868 vdd vdd pch w=2u l=180n
CT872 t872 0 0.1f
M2407 nw332 t867 t872 0 nch w=1u l=180n
M2408 t872 t868 0 0 nch w=1u l=180n
Cnw332 nw332 0 2f
M2409 nw333 nw145 vdd vdd pch w=2u l=180n
M2410 nw333 nw39 vdd vdd pch w=2u l=180n
CT873 t873 0 0.1f
M2411 nw333 nw145 t873 0 nch w=1u l=180n
M2412 t873 nw39 0 0 nch w=1u l=180n
Cnw333 nw333 0 2f
M2413 nw334 nw146 0 0 nch w=1u l=180n
M2414 nw334 nw40 0 0 nch w=1u l=180n
CT874 t874 0 0.1f
M2415 t874 nw146 vdd vdd pch w=2u l=180n
M2416 nw334 nw40 t874 vdd pch w=2u l=180n
Cnw334 nw334 0 2f
CT875 t875 0 0.1f
M2417 t875 nw147 vdd vdd pch w=2u l=180n
M2418 t875 nw41 vdd vdd pch w=2u l=180n
CT876 t876 0 0.1f
M2419 t875 nw147 t876 0 nch w=1u l=180n
M2420 t876 nw41 0 0 nch w=1u l=180n
M2421 nw335 t875 vdd vdd pch w=2u l=180n
M2422 nw335 t875 0 0 nch w=1u l=180n
Cnw335 nw335 0 2f
CT877 t877 0 0.1f
M2423 t877 nw148 0 0 nch w=1u l=180n
M2424 t877 nw42 0 0 nch w=1u l=180n
CT878 t878 0 0.1f
M2425 t878 nw148 vdd vdd pch w=2u l=180n
M2426 t877 nw42 t878 vdd pch w=2u l=180n
M2427 nw336 t877 vdd vdd pch w=2u l=180n
M2428 nw336 t877 0 0 nch w=1u l=180n
Cnw336 nw336 0 2f
CT879 t879 0 0.1f
CT880 t880 0 0.1f
CT881 t881 0 0.1f
M2429 t879 nw149 vdd vdd pch w=2u l=180n
M2430 t879 nw43 vdd vdd pch w=2u l=180n
CT882 t882 0 0.1f
M2431 t879 nw149 t882 0 nch w=1u l=180n
M2432 t882 nw43 0 0 nch w=1u l=180n
M2433 t880 nw149 vdd vdd pch w=2u l=180n
M2434 t880 t879 vdd vdd pch w=2u l=180n
CT883 t883 0 0.1f
M2435 t880 nw149 t883 0 nch w=1u l=180n
M2436 t883 t879 0 0 nch w=1u l=180n
M2437 t881 nw43 vdd vdd pch w=2u l=180n
M2438 t881 t879 vdd vdd pch w=2u l=180n
CT884 t884 0 0.1f
M2439 t881 nw43 t884 0 nch w=1u l=180n
M2440 t884 t879 0 0 nch w=1u l=180n
M2441 nw337 t880 vdd vdd pch w=2u l=180n
M2442 nw337 t881 vdd vdd pch w=2u l=180n
CT885 t885 0 0.1f
M2443 nw337 t880 t885 0 nch w=1u l=180n
M2444 t885 t881 0 0 nch w=1u l=180n
Cnw337 nw337 0 2f
M2445 nw338 nw150 vdd vdd pch w=2u l=180n
M2446 nw338 nw44 vdd vdd pch w=2u l=180n
CT886 t886 0 0.1f
M2447 nw338 nw150 t886 0 nch w=1u l=180n
M2448 t886 nw44 0 0 nch w=1u l=180n
Cnw338 nw338 0 2f
M2449 nw339 nw151 0 0 nch w=1u l=180n
M2450 nw339 nw45 0 0 nch w=1u l=180n
CT887 t887 0 0.1f
M2451 t887 nw151 vdd vdd pch w=2u l=180n
M2452 nw339 nw45 t887 vdd pch w=2u l=180n
Cnw339 nw339 0 2f
CT888 t888 0 0.1f
M2453 t888 nw152 vdd vdd pch w=2u l=180n
M2454 t888 nw46 vdd vdd pch w=2u l=180n
CT889 t889 0 0.1f
M2455 t888 nw152 t889 0 nch w=1u l=180n
M2456 t889 nw46 0 0 nch w=1u l=180n
M2457 nw340 t888 vdd vdd pch w=2u l=180n
M2458 nw340 t888 0 0 nch w=1u l=180n
Cnw340 nw340 0 2f
CT890 t890 0 0.1f
M2459 t890 nw153 0 0 nch w=1u l=180n
M2460 t890 nw47 0 0 nch w=1u l=180n
CT891 t891 0 0.1f
M2461 t891 nw153 vdd vdd pch w=2u l=180n
M2462 t890 nw47 t891 vdd pch w=2u l=180n
M2463 nw341 t890 vdd vdd pch w=2u l=180n
M2464 nw341 t890 0 0 nch w=1u l=180n
Cnw341 nw341 0 2f
CT892 t892 0 0.1f
CT893 t893 0 0.1f
CT894 t894 0 0.1f
M2465 t892 nw154 vdd vdd pch w=2u l=180n
M2466 t892 nw48 vdd vdd pch w=2u l=180n
CT895 t895 0 0.1f
M2467 t892 nw154 t895 0 nch w=1u l=180n
M2468 t895 nw48 0 0 nch w=1u l=180n
M2469 t893 nw154 vdd vdd pch w=2u l=180n
M2470 t893 t892 vdd vdd pch w=2u l=180n
CT896 t896 0 0.1f
M2471 t893 nw154 t896 0 nch w=1u l=180n
M2472 t896 t892 0 0 nch w=1u l=180n
M2473 t894 nw48 vdd vdd pch w=2u l=180n
M2474 t894 t892 vdd vdd pch w=2u l=180n
CT897 t897 0 0.1f
M2475 t894 nw48 t897 0 nch w=1u l=180n
M2476 t897 t892 0 0 nch w=1u l=180n
M2477 nw342 t893 vdd vdd pch w=2u l=180n
M2478 nw342 t894 vdd vdd pch w=2u l=180n
CT898 t898 0 0.1f
M2479 nw342 t893 t898 0 nch w=1u l=180n
M2480 t898 t894 0 0 nch w=1u l=180n
Cnw342 nw342 0 2f
M2481 nw343 nw155 vdd vdd pch w=2u l=180n
M2482 nw343 nw49 vdd vdd pch w=2u l=180n
CT899 t899 0 0.1f
M2483 nw343 nw155 t899 0 nch w=1u l=180n
M2484 t899 nw49 0 0 nch w=1u l=180n
Cnw343 nw343 0 2f
M2485 nw344 nw156 0 0 nch w=1u l=180n
M2486 nw344 nw50 0 0 nch w=1u l=180n
CT900 t900 0 0.1f
M2487 t900 nw156 vdd vdd pch w=2u l=180n
M2488 nw344 nw50 t900 vdd pch w=2u l=180n
Cnw344 nw344 0 2f
CT901 t901 0 0.1f
M2489 t901 nw157 vdd vdd pch w=2u l=180n
M2490 t901 nw51 vdd vdd pch w=2u l=180n
CT902 t902 0 0.1f
M2491 t901 nw157 t902 0 nch w=1u l=180n
M2492 t902 nw51 0 0 nch w=1u l=180n
M2493 nw345 t901 vdd vdd pch w=2u l=180n
M2494 nw345 t901 0 0 nch w=1u l=180n
Cnw345 nw345 0 2f
CT903 t903 0 0.1f
M2495 t903 nw158 0 0 nch w=1u l=180n
M2496 t903 nw52 0 0 nch w=1u l=180n
CT904 t904 0 0.1f
M2497 t904 nw158 vdd vdd pch w=2u l=180n
M2498 t903 nw52 t904 vdd pch w=2u l=180n
M2499 nw346 t903 vdd vdd pch w=2u l=180n
M2500 nw346 t903 0 0 nch w=1u l=180n
Cnw346 nw346 0 2f
CT905 t905 0 0.1f
CT906 t906 0 0.1f
CT907 t907 0 0.1f
M2501 t905 nw159 vdd vdd pch w=2u l=180n
M2502 t905 nw53 vdd vdd pch w=2u l=180n
CT908 t908 0 0.1f
M2503 t905 nw159 t908 0 nch w=1u l=180n
M2504 t908 nw53 0 0 nch w=1u l=180n
M2505 t906 nw159 vdd vdd pch w=2u l=180n
M2506 t906 t905 vdd vdd pch w=2u l=180n
CT909 t909 0 0.1f
M2507 t906 nw159 t909 0 nch w=1u l=180n
M2508 t909 t905 0 0 nch w=1u l=180n
M2509 t907 nw53 vdd vdd pch w=2u l=180n
M2510 t907 t905 vdd vdd pch w=2u l=180n
CT910 t910 0 0.1f
M2511 t907 nw53 t910 0 nch w=1u l=180n
M2512 t910 t905 0 0 nch w=1u l=180n
M2513 nw347 t906 vdd vdd pch w=2u l=180n
M2514 nw347 t907 vdd vdd pch w=2u l=180n
CT911 t911 0 0.1f
M2515 nw347 t906 t911 0 nch w=1u l=180n
M2516 t911 t907 0 0 nch w=1u l=180n
Cnw347 nw347 0 2f
M2517 nw348 nw160 vdd vdd pch w=2u l=180n
M2518 nw348 nw54 vdd vdd pch w=2u l=180n
CT912 t912 0 0.1f
M2519 nw348 nw160 t912 0 nch w=1u l=180n
M2520 t912 nw54 0 0 nch w=1u l=180n
Cnw348 nw348 0 2f
M2521 nw349 nw161 0 0 nch w=1u l=180n
M2522 nw349 nw55 0 0 nch w=1u l=180n
CT913 t913 0 0.1f
M2523 t913 nw161 vdd vdd pch w=2u l=180n
M2524 nw349 nw55 t913 vdd pch w=2u l=180n
Cnw349 nw349 0 2f
CT914 t914 0 0.1f
M2525 t914 nw162 vdd vdd pch w=2u l=180n
M2526 t914 nw56 vdd vdd pch w=2u l=180n
CT915 t915 0 0.1f
M2527 t914 nw162 t915 0 nch w=1u l=180n
M2528 t915 nw56 0 0 nch w=1u l=180n
M2529 nw350 t914 vdd vdd pch w=2u l=180n
M2530 nw350 t914 0 0 nch w=1u l=180n
Cnw350 nw350 0 2f
CT916 t916 0 0.1f
M2531 t916 nw163 0 0 nch w=1u l=180n
M2532 t916 nw57 0 0 nch w=1u l=180n
CT917 t917 0 0.1f
M2533 t917 nw163 vdd vdd pch w=2u l=180n
M2534 t916 nw57 t917 vdd pch w=2u l=180n
M2535 nw351 t916 vdd vdd pch w=2u l=180n
M2536 nw351 t916 0 0 nch w=1u l=180n
Cnw351 nw351 0 2f
CT918 t918 0 0.1f
CT919 t919 0 0.1f
CT920 t920 0 0.1f
M2537 t918 nw164 vdd vdd pch w=2u l=180n
M2538 t918 nw58 vdd vdd pch w=2u l=180n
CT921 t921 0 0.1f
M2539 t918 nw164 t921 0 nch w=1u l=180n
M2540 t921 nw58 0 0 nch w=1u l=180n
M2541 t919 nw164 vdd vdd pch w=2u l=180n
M2542 t919 t918 vdd vdd pch w=2u l=180n
CT922 t922 0 0.1f
M2543 t919 nw164 t922 0 nch w=1u l=180n
M2544 t922 t918 0 0 nch w=1u l=180n
M2545 t920 nw58 vdd vdd pch w=2u l=180n
M2546 t920 t918 vdd vdd pch w=2u l=180n
CT923 t923 0 0.1f
M2547 t920 nw58 t923 0 nch w=1u l=180n
M2548 t923 t918 0 0 nch w=1u l=180n
M2549 nw352 t919 vdd vdd pch w=2u l=180n
M2550 nw352 t920 vdd vdd pch w=2u l=180n
CT924 t924 0 0.1f
M2551 nw352 t919 t924 0 nch w=1u l=180n
M2552 t924 t920 0 0 nch w=1u l=180n
Cnw352 nw352 0 2f
M2553 nw353 nw165 vdd vdd pch w=2u l=180n
M2554 nw353 nw59 vdd vdd pch w=2u l=180n
CT925 t925 0 0.1f
M2555 nw353 nw165 t925 0 nch w=1u l=180n
M2556 t925 nw59 0 0 nch w=1u l=180n
Cnw353 nw353 0 2f
M2557 nw354 nw166 0 0 nch w=1u l=180n
M2558 nw354 nw60 0 0 nch w=1u l=180n
CT926 t926 0 0.1f
M2559 t926 nw166 vdd vdd pch w=2u l=180n
M2560 nw354 nw60 t926 vdd pch w=2u l=180n
Cnw354 nw354 0 2f
CT927 t927 0 0.1f
M2561 t927 nw167 vdd vdd pch w=2u l=180n
M2562 t927 nw61 vdd vdd pch w=2u l=180n
CT928 t928 0 0.1f
M2563 t927 nw167 t928 0 nch w=1u l=180n
M2564 t928 nw61 0 0 nch w=1u l=180n
M2565 nw355 t927 vdd vdd pch w=2u l=180n
M2566 nw355 t927 0 0 nch w=1u l=180n
Cnw355 nw355 0 2f
CT929 t929 0 0.1f
M2567 t929 nw168 0 0 nch w=1u l=180n
M2568 t929 nw62 0 0 nch w=1u l=180n
CT930 t930 0 0.1f
M2569 t930 nw168 vdd vdd pch w=2u l=180n
M2570 t929 nw62 t930 vdd pch w=2u l=180n
M2571 nw356 t929 vdd vdd pch w=2u l=180n
M2572 nw356 t929 0 0 nch w=1u l=180n
Cnw356 nw356 0 2f
CT931 t931 0 0.1f
CT932 t932 0 0.1f
CT933 t933 0 0.1f
M2573 t931 nw169 vdd vdd pch w=2u l=180n
M2574 t931 nw63 vdd vdd pch w=2u l=180n
CT934 t934 0 0.1f
M2575 t931 nw169 t934 0 nch w=1u l=180n
M2576 t934 nw63 0 0 nch w=1u l=180n
M2577 t932 nw169 vdd vdd pch w=2u l=180n
M2578 t932 t931 vdd vdd pch w=2u l=180n
CT935 t935 0 0.1f
M2579 t932 nw169 t935 0 nch w=1u l=180n
M2580 t935 t931 0 0 nch w=1u l=180n
M2581 t933 nw63 vdd vdd pch w=2u l=180n
M2582 t933 t931 vdd vdd pch w=2u l=180n
CT936 t936 0 0.1f
M2583 t933 nw63 t936 0 nch w=1u l=180n
M2584 t936 t931 0 0 nch w=1u l=180n
M2585 nw357 t932 vdd vdd pch w=2u l=180n
M2586 nw357 t933 vdd vdd pch w=2u l=180n
CT937 t937 0 0.1f
M2587 nw357 t932 t937 0 nch w=1u l=180n
M2588 t937 t933 0 0 nch w=1u l=180n
Cnw357 nw357 0 2f
M2589 nw358 nw170 vdd vdd pch w=2u l=180n
M2590 nw358 nw64 vdd vdd pch w=2u l=180n
CT938 t938 0 0.1f
M2591 nw358 nw170 t938 0 nch w=1u l=180n
M2592 t938 nw64 0 0 nch w=1u l=180n
Cnw358 nw358 0 2f
M2593 nw359 nw171 0 0 nch w=1u l=180n
M2594 nw359 nw65 0 0 nch w=1u l=180n
CT939 t939 0 0.1f
M2595 t939 nw171 vdd vdd pch w=2u l=180n
M2596 nw359 nw65 t939 vdd pch w=2u l=180n
Cnw359 nw359 0 2f
CT940 t940 0 0.1f
M2597 t940 nw172 vdd vdd pch w=2u l=180n
M2598 t940 nw66 vdd vdd pch w=2u l=180n
CT941 t941 0 0.1f
M2599 t940 nw172 t941 0 nch w=1u l=180n
M2600 t941 nw66 0 0 nch w=1u l=180n
M2601 nw360 t940 vdd vdd pch w=2u l=180n
M2602 nw360 t940 0 0 nch w=1u l=180n
Cnw360 nw360 0 2f
CT942 t942 0 0.1f
M2603 t942 nw173 0 0 nch w=1u l=180n
M2604 t942 nw67 0 0 nch w=1u l=180n
CT943 t943 0 0.1f
M2605 t943 nw173 vdd vdd pch w=2u l=180n
M2606 t942 nw67 t943 vdd pch w=2u l=180n
M2607 nw361 t942 vdd vdd pch w=2u l=180n
M2608 nw361 t942 0 0 nch w=1u l=180n
Cnw361 nw361 0 2f
CT944 t944 0 0.1f
CT945 t945 0 0.1f
CT946 t946 0 0.1f
M2609 t944 nw174 vdd vdd pch w=2u l=180n
M2610 t944 nw68 vdd vdd pch w=2u l=180n
CT947 t947 0 0.1f
M2611 t944 nw174 t947 0 nch w=1u l=180n
M2612 t947 nw68 0 0 nch w=1u l=180n
M2613 t945 nw174 vdd vdd pch w=2u l=180n
M2614 t945 t944 vdd vdd pch w=2u l=180n
CT948 t948 0 0.1f
M2615 t945 nw174 t948 0 nch w=1u l=180n
M2616 t948 t944 0 0 nch w=1u l=180n
M2617 t946 nw68 vdd vdd pch w=2u l=180n
M2618 t946 t944 vdd vdd pch w=2u l=180n
CT949 t949 0 0.1f
M2619 t946 nw68 t949 0 nch w=1u l=180n
M2620 t949 t944 0 0 nch w=1u l=180n
M2621 nw362 t945 vdd vdd pch w=2u l=180n
M2622 nw362 t946 vdd vdd pch w=2u l=180n
CT950 t950 0 0.1f
M2623 nw362 t945 t950 0 nch w=1u l=180n
M2624 t950 t946 0 0 nch w=1u l=180n
Cnw362 nw362 0 2f
M2625 nw363 nw175 vdd vdd pch w=2u l=180n
M2626 nw363 nw69 vdd vdd pch w=2u l=180n
CT951 t951 0 0.1f
M2627 nw363 nw175 t951 0 nch w=1u l=180n
M2628 t951 nw69 0 0 nch w=1u l=180n
Cnw363 nw363 0 2f
M2629 nw364 nw176 0 0 nch w=1u l=180n
M2630 nw364 nw70 0 0 nch w=1u l=180n
CT952 t952 0 0.1f
M2631 t952 nw176 vdd vdd pch w=2u l=180n
M2632 nw364 nw70 t952 vdd pch w=2u l=180n
Cnw364 nw364 0 2f
CT953 t953 0 0.1f
M2633 t953 nw177 vdd vdd pch w=2u l=180n
M2634 t953 nw71 vdd vdd pch w=2u l=180n
CT954 t954 0 0.1f
M2635 t953 nw177 t954 0 nch w=1u l=180n
M2636 t954 nw71 0 0 nch w=1u l=180n
M2637 nw365 t953 vdd vdd pch w=2u l=180n
M2638 nw365 t953 0 0 nch w=1u l=180n
Cnw365 nw365 0 2f
CT955 t955 0 0.1f
M2639 t955 nw178 0 0 nch w=1u l=180n
M2640 t955 nw72 0 0 nch w=1u l=180n
CT956 t956 0 0.1f
M2641 t956 nw178 vdd vdd pch w=2u l=180n
M2642 t955 nw72 t956 vdd pch w=2u l=180n
M2643 nw366 t955 vdd vdd pch w=2u l=180n
M2644 nw366 t955 0 0 nch w=1u l=180n
Cnw366 nw366 0 2f
CT957 t957 0 0.1f
CT958 t958 0 0.1f
CT959 t959 0 0.1f
M2645 t957 nw179 vdd vdd pch w=2u l=180n
M2646 t957 nw73 vdd vdd pch w=2u l=180n
CT960 t960 0 0.1f
M2647 t957 nw179 t960 0 nch w=1u l=180n
M2648 t960 nw73 0 0 nch w=1u l=180n
M2649 t958 nw179 vdd vdd pch w=2u l=180n
M2650 t958 t957 vdd vdd pch w=2u l=180n
CT961 t961 0 0.1f
M2651 t958 nw179 t961 0 nch w=1u l=180n
M2652 t961 t957 0 0 nch w=1u l=180n
M2653 t959 nw73 vdd vdd pch w=2u l=180n
M2654 t959 t957 vdd vdd pch w=2u l=180n
CT962 t962 0 0.1f
M2655 t959 nw73 t962 0 nch w=1u l=180n
M2656 t962 t957 0 0 nch w=1u l=180n
M2657 nw367 t958 vdd vdd pch w=2u l=180n
M2658 nw367 t959 vdd vdd pch w=2u l=180n
CT963 t963 0 0.1f
M2659 nw367 t958 t963 0 nch w=1u l=180n
M2660 t963 t959 0 0 nch w=1u l=180n
Cnw367 nw367 0 2f
M2661 nw368 nw180 vdd vdd pch w=2u l=180n
M2662 nw368 nw74 vdd vdd pch w=2u l=180n
CT964 t964 0 0.1f
M2663 nw368 nw180 t964 0 nch w=1u l=180n
M2664 t964 nw74 0 0 nch w=1u l=180n
Cnw368 nw368 0 2f
M2665 nw369 nw181 0 0 nch w=1u l=180n
M2666 nw369 nw75 0 0 nch w=1u l=180n
CT965 t965 0 0.1f
M2667 t965 nw181 vdd vdd pch w=2u l=180n
M2668 nw369 nw75 t965 vdd pch w=2u l=180n
Cnw369 nw369 0 2f
CT966 t966 0 0.1f
M2669 t966 nw182 vdd vdd pch w=2u l=180n
M2670 t966 nw76 vdd vdd pch w=2u l=180n
CT967 t967 0 0.1f
M2671 t966 nw182 t967 0 nch w=1u l=180n
M2672 t967 nw76 0 0 nch w=1u l=180n
M2673 nw370 t966 vdd vdd pch w=2u l=180n
M2674 nw370 t966 0 0 nch w=1u l=180n
Cnw370 nw370 0 2f
CT968 t968 0 0.1f
M2675 t968 nw183 0 0 nch w=1u l=180n
M2676 t968 nw77 0 0 nch w=1u l=180n
CT969 t969 0 0.1f
M2677 t969 nw183 vdd vdd pch w=2u l=180n
M2678 t968 nw77 t969 vdd pch w=2u l=180n
M2679 nw371 t968 vdd vdd pch w=2u l=180n
M2680 nw371 t968 0 0 nch w=1u l=180n
Cnw371 nw371 0 2f
CT970 t970 0 0.1f
CT971 t971 0 0.1f
CT972 t972 0 0.1f
M2681 t970 nw184 vdd vdd pch w=2u l=180n
M2682 t970 nw78 vdd vdd pch w=2u l=180n
CT973 t973 0 0.1f
M2683 t970 nw184 t973 0 nch w=1u l=180n
M2684 t973 nw78 0 0 nch w=1u l=180n
M2685 t971 nw184 vdd vdd pch w=2u l=180n
M2686 t971 t970 vdd vdd pch w=2u l=180n
CT974 t974 0 0.1f
M2687 t971 nw184 t974 0 nch w=1u l=180n
M2688 t974 t970 0 0 nch w=1u l=180n
M2689 t972 nw78 vdd vdd pch w=2u l=180n
M2690 t972 t970 vdd vdd pch w=2u l=180n
CT975 t975 0 0.1f
M2691 t972 nw78 t975 0 nch w=1u l=180n
M2692 t975 t970 0 0 nch w=1u l=180n
M2693 nw372 t971 vdd vdd pch w=2u l=180n
M2694 nw372 t972 vdd vdd pch w=2u l=180n
CT976 t976 0 0.1f
M2695 nw372 t971 t976 0 nch w=1u l=180n
M2696 t976 t972 0 0 nch w=1u l=180n
Cnw372 nw372 0 2f
M2697 nw373 nw185 vdd vdd pch w=2u l=180n
M2698 nw373 nw79 vdd vdd pch w=2u l=180n
CT977 t977 0 0.1f
M2699 nw373 nw185 t977 0 nch w=1u l=180n
M2700 t977 nw79 0 0 nch w=1u l=180n
Cnw373 nw373 0 2f
M2701 nw374 nw186 0 0 nch w=1u l=180n
M2702 nw374 nw80 0 0 nch w=1u l=180n
CT978 t978 0 0.1f
M2703 t978 nw186 vdd vdd pch w=2u l=180n
M2704 nw374 nw80 t978 vdd pch w=2u l=180n
Cnw374 nw374 0 2f
CT979 t979 0 0.1f
M2705 t979 nw187 vdd vdd pch w=2u l=180n
M2706 t979 nw81 vdd vdd pch w=2u l=180n
CT980 t980 0 0.1f
M2707 t979 nw187 t980 0 nch w=1u l=180n
M2708 t980 nw81 0 0 nch w=1u l=180n
M2709 nw375 t979 vdd vdd pch w=2u l=180n
M2710 nw375 t979 0 0 nch w=1u l=180n
Cnw375 nw375 0 2f
CT981 t981 0 0.1f
M2711 t981 nw188 0 0 nch w=1u l=180n
M2712 t981 nw82 0 0 nch w=1u l=180n
CT982 t982 0 0.1f
M2713 t982 nw188 vdd vdd pch w=2u l=180n
M2714 t981 nw82 t982 vdd pch w=2u l=180n
M2715 nw376 t981 vdd vdd pch w=2u l=180n
M2716 nw376 t981 0 0 nch w=1u l=180n
Cnw376 nw376 0 2f
CT983 t983 0 0.1f
CT984 t984 0 0.1f
CT985 t985 0 0.1f
M2717 t983 nw189 vdd vdd pch w=2u l=180n
M2718 t983 nw83 vdd vdd pch w=2u l=180n
CT986 t986 0 0.1f
M2719 t983 nw189 t986 0 nch w=1u l=180n
M2720 t986 nw83 0 0 nch w=1u l=180n
M2721 t984 nw189 vdd vdd pch w=2u l=180n
M2722 t984 t983 vdd vdd pch w=2u l=180n
CT987 t987 0 0.1f
M2723 t984 nw189 t987 0 nch w=1u l=180n
M2724 t987 t983 0 0 nch w=1u l=180n
M2725 t985 nw83 vdd vdd pch w=2u l=180n
M2726 t985 t983 vdd vdd pch w=2u l=180n
CT988 t988 0 0.1f
M2727 t985 nw83 t988 0 nch w=1u l=180n
M2728 t988 t983 0 0 nch w=1u l=180n
M2729 nw377 t984 vdd vdd pch w=2u l=180n
M2730 nw377 t985 vdd vdd pch w=2u l=180n
CT989 t989 0 0.1f
M2731 nw377 t984 t989 0 nch w=1u l=180n
M2732 t989 t985 0 0 nch w=1u l=180n
Cnw377 nw377 0 2f
M2733 nw378 nw190 vdd vdd pch w=2u l=180n
M2734 nw378 nw84 vdd vdd pch w=2u l=180n
CT990 t990 0 0.1f
M2735 nw378 nw190 t990 0 nch w=1u l=180n
M2736 t990 nw84 0 0 nch w=1u l=180n
Cnw378 nw378 0 2f
M2737 nw379 nw191 0 0 nch w=1u l=180n
M2738 nw379 nw85 0 0 nch w=1u l=180n
CT991 t991 0 0.1f
M2739 t991 nw191 vdd vdd pch w=2u l=180n
M2740 nw379 nw85 t991 vdd pch w=2u l=180n
Cnw379 nw379 0 2f
CT992 t992 0 0.1f
M2741 t992 nw192 vdd vdd pch w=2u l=180n
M2742 t992 nw86 vdd vdd pch w=2u l=180n
CT993 t993 0 0.1f
M2743 t992 nw192 t993 0 nch w=1u l=180n
M2744 t993 nw86 0 0 nch w=1u l=180n
M2745 nw380 t992 vdd vdd pch w=2u l=180n
M2746 nw380 t992 0 0 nch w=1u l=180n
Cnw380 nw380 0 2f
CT994 t994 0 0.1f
M2747 t994 nw193 0 0 nch w=1u l=180n
M2748 t994 nw87 0 0 nch w=1u l=180n
CT995 t995 0 0.1f
M2749 t995 nw193 vdd vdd pch w=2u l=180n
M2750 t994 nw87 t995 vdd pch w=2u l=180n
M2751 nw381 t994 vdd vdd pch w=2u l=180n
M2752 nw381 t994 0 0 nch w=1u l=180n
Cnw381 nw381 0 2f
CT996 t996 0 0.1f
CT997 t997 0 0.1f
CT998 t998 0 0.1f
M2753 t996 nw194 vdd vdd pch w=2u l=180n
M2754 t996 nw88 vdd vdd pch w=2u l=180n
CT999 t999 0 0.1f
M2755 t996 nw194 t999 0 nch w=1u l=180n
M2756 t999 nw88 0 0 nch w=1u l=180n
M2757 t997 nw194 vdd vdd pch w=2u l=180n
M2758 t997 t996 vdd vdd pch w=2u l=180n
CT1000 t1000 0 0.1f
M2759 t997 nw194 t1000 0 nch w=1u l=180n
M2760 t1000 t996 0 0 nch w=1u l=180n
M2761 t998 nw88 vdd vdd pch w=2u l=180n
M2762 t998 t996 vdd vdd pch w=2u l=180n
CT1001 t1001 0 0.1f
M2763 t998 nw88 t1001 0 nch w=1u l=180n
M2764 t1001 t996 0 0 nch w=1u l=180n
M2765 nw382 t997 vdd vdd pch w=2u l=180n
M2766 nw382 t998 vdd vdd pch w=2u l=180n
CT1002 t1002 0 0.1f
M2767 nw382 t997 t1002 0 nch w=1u l=180n
M2768 t1002 t998 0 0 nch w=1u l=180n
Cnw382 nw382 0 2f
M2769 nw383 nw195 vdd vdd pch w=2u l=180n
M2770 nw383 nw89 vdd vdd pch w=2u l=180n
CT1003 t1003 0 0.1f
M2771 nw383 nw195 t1003 0 nch w=1u l=180n
M2772 t1003 nw89 0 0 nch w=1u l=180n
Cnw383 nw383 0 2f
M2773 nw384 nw196 0 0 nch w=1u l=180n
M2774 nw384 nw90 0 0 nch w=1u l=180n
CT1004 t1004 0 0.1f
M2775 t1004 nw196 vdd vdd pch w=2u l=180n
M2776 nw384 nw90 t1004 vdd pch w=2u l=180n
Cnw384 nw384 0 2f
CT1005 t1005 0 0.1f
M2777 t1005 nw197 vdd vdd pch w=2u l=180n
M2778 t1005 nw91 vdd vdd pch w=2u l=180n
CT1006 t1006 0 0.1f
M2779 t1005 nw197 t1006 0 nch w=1u l=180n
M2780 t1006 nw91 0 0 nch w=1u l=180n
M2781 nw385 t1005 vdd vdd pch w=2u l=180n
M2782 nw385 t1005 0 0 nch w=1u l=180n
Cnw385 nw385 0 2f
CT1007 t1007 0 0.1f
M2783 t1007 nw198 0 0 nch w=1u l=180n
M2784 t1007 nw92 0 0 nch w=1u l=180n
CT1008 t1008 0 0.1f
M2785 t1008 nw198 vdd vdd pch w=2u l=180n
M2786 t1007 nw92 t1008 vdd pch w=2u l=180n
M2787 nw386 t1007 vdd vdd pch w=2u l=180n
M2788 nw386 t1007 0 0 nch w=1u l=180n
Cnw386 nw386 0 2f
CT1009 t1009 0 0.1f
CT1010 t1010 0 0.1f
CT1011 t1011 0 0.1f
M2789 t1009 nw199 vdd vdd pch w=2u l=180n
M2790 t1009 nw93 vdd vdd pch w=2u l=180n
CT1012 t1012 0 0.1f
M2791 t1009 nw199 t1012 0 nch w=1u l=180n
M2792 t1012 nw93 0 0 nch w=1u l=180n
M2793 t1010 nw199 vdd vdd pch w=2u l=180n
M2794 t1010 t1009 vdd vdd pch w=2u l=180n
CT1013 t1013 0 0.1f
M2795 t1010 nw199 t1013 0 nch w=1u l=180n
M2796 t1013 t1009 0 0 nch w=1u l=180n
M2797 t1011 nw93 vdd vdd pch w=2u l=180n
M2798 t1011 t1009 vdd vdd pch w=2u l=180n
CT1014 t1014 0 0.1f
M2799 t1011 nw93 t1014 0 nch w=1u l=180n
M2800 t1014 t1009 0 0 nch w=1u l=180n
M2801 nw387 t1010 vdd vdd pch w=2u l=180n
M2802 nw387 t1011 vdd vdd pch w=2u l=180n
CT1015 t1015 0 0.1f
M2803 nw387 t1010 t1015 0 nch w=1u l=180n
M2804 t1015 t1011 0 0 nch w=1u l=180n
Cnw387 nw387 0 2f
M2805 nw388 nw200 vdd vdd pch w=2u l=180n
M2806 nw388 nw94 vdd vdd pch w=2u l=180n
CT1016 t1016 0 0.1f
M2807 nw388 nw200 t1016 0 nch w=1u l=180n
M2808 t1016 nw94 0 0 nch w=1u l=180n
Cnw388 nw388 0 2f
M2809 nw389 nw201 0 0 nch w=1u l=180n
M2810 nw389 nw95 0 0 nch w=1u l=180n
CT1017 t1017 0 0.1f
M2811 t1017 nw201 vdd vdd pch w=2u l=180n
M2812 nw389 nw95 t1017 vdd pch w=2u l=180n
Cnw389 nw389 0 2f
CT1018 t1018 0 0.1f
M2813 t1018 nw202 vdd vdd pch w=2u l=180n
M2814 t1018 nw96 vdd vdd pch w=2u l=180n
CT1019 t1019 0 0.1f
M2815 t1018 nw202 t1019 0 nch w=1u l=180n
M2816 t1019 nw96 0 0 nch w=1u l=180n
M2817 nw390 t1018 vdd vdd pch w=2u l=180n
M2818 nw390 t1018 0 0 nch w=1u l=180n
Cnw390 nw390 0 2f
CT1020 t1020 0 0.1f
M2819 t1020 nw203 0 0 nch w=1u l=180n
M2820 t1020 nw97 0 0 nch w=1u l=180n
CT1021 t1021 0 0.1f
M2821 t1021 nw203 vdd vdd pch w=2u l=180n
M2822 t1020 nw97 t1021 vdd pch w=2u l=180n
M2823 nw391 t1020 vdd vdd pch w=2u l=180n
M2824 nw391 t1020 0 0 nch w=1u l=180n
Cnw391 nw391 0 2f
CT1022 t1022 0 0.1f
CT1023 t1023 0 0.1f
CT1024 t1024 0 0.1f
M2825 t1022 nw204 vdd vdd pch w=2u l=180n
M2826 t1022 nw98 vdd vdd pch w=2u l=180n
CT1025 t1025 0 0.1f
M2827 t1022 nw204 t1025 0 nch w=1u l=180n
M2828 t1025 nw98 0 0 nch w=1u l=180n
M2829 t1023 nw204 vdd vdd pch w=2u l=180n
M2830 t1023 t1022 vdd vdd pch w=2u l=180n
CT1026 t1026 0 0.1f
M2831 t1023 nw204 t1026 0 nch w=1u l=180n
M2832 t1026 t1022 0 0 nch w=1u l=180n
M2833 t1024 nw98 vdd vdd pch w=2u l=180n
M2834 t1024 t1022 vdd vdd pch w=2u l=180n
CT1027 t1027 0 0.1f
M2835 t1024 nw98 t1027 0 nch w=1u l=180n
M2836 t1027 t1022 0 0 nch w=1u l=180n
M2837 nw392 t1023 vdd vdd pch w=2u l=180n
M2838 nw392 t1024 vdd vdd pch w=2u l=180n
CT1028 t1028 0 0.1f
M2839 nw392 t1023 t1028 0 nch w=1u l=180n
M2840 t1028 t1024 0 0 nch w=1u l=180n
Cnw392 nw392 0 2f
M2841 nw393 nw205 vdd vdd pch w=2u l=180n
M2842 nw393 nw99 vdd vdd pch w=2u l=180n
CT1029 t1029 0 0.1f
M2843 nw393 nw205 t1029 0 nch w=1u l=180n
M2844 t1029 nw99 0 0 nch w=1u l=180n
Cnw393 nw393 0 2f
M2845 nw394 nw206 0 0 nch w=1u l=180n
M2846 nw394 nw100 0 0 nch w=1u l=180n
CT1030 t1030 0 0.1f
M2847 t1030 nw206 vdd vdd pch w=2u l=180n
M2848 nw394 nw100 t1030 vdd pch w=2u l=180n
Cnw394 nw394 0 2f
CT1031 t1031 0 0.1f
M2849 t1031 nw207 vdd vdd pch w=2u l=180n
M2850 t1031 nw101 vdd vdd pch w=2u l=180n
CT1032 t1032 0 0.1f
M2851 t1031 nw207 t1032 0 nch w=1u l=180n
M2852 t1032 nw101 0 0 nch w=1u l=180n
M2853 nw395 t1031 vdd vdd pch w=2u l=180n
M2854 nw395 t1031 0 0 nch w=1u l=180n
Cnw395 nw395 0 2f
CT1033 t1033 0 0.1f
M2855 t1033 nw208 0 0 nch w=1u l=180n
M2856 t1033 nw102 0 0 nch w=1u l=180n
CT1034 t1034 0 0.1f
M2857 t1034 nw208 vdd vdd pch w=2u l=180n
M2858 t1033 nw102 t1034 vdd pch w=2u l=180n
M2859 nw396 t1033 vdd vdd pch w=2u l=180n
M2860 nw396 t1033 0 0 nch w=1u l=180n
Cnw396 nw396 0 2f
CT1035 t1035 0 0.1f
CT1036 t1036 0 0.1f
CT1037 t1037 0 0.1f
M2861 t1035 nw209 vdd vdd pch w=2u l=180n
M2862 t1035 nw103 vdd vdd pch w=2u l=180n
CT1038 t1038 0 0.1f
M2863 t1035 nw209 t1038 0 nch w=1u l=180n
M2864 t1038 nw103 0 0 nch w=1u l=180n
M2865 t1036 nw209 vdd vdd pch w=2u l=180n
M2866 t1036 t1035 vdd vdd pch w=2u l=180n
CT1039 t1039 0 0.1f
M2867 t1036 nw209 t1039 0 nch w=1u l=180n
M2868 t1039 t1035 0 0 nch w=1u l=180n
M2869 t1037 nw103 vdd vdd pch w=2u l=180n
M2870 t1037 t1035 vdd vdd pch w=2u l=180n
CT1040 t1040 0 0.1f
M2871 t1037 nw103 t1040 0 nch w=1u l=180n
M2872 t1040 t1035 0 0 nch w=1u l=180n
M2873 nw397 t1036 vdd vdd pch w=2u l=180n
M2874 nw397 t1037 vdd vdd pch w=2u l=180n
CT1041 t1041 0 0.1f
M2875 nw397 t1036 t1041 0 nch w=1u l=180n
M2876 t1041 t1037 0 0 nch w=1u l=180n
Cnw397 nw397 0 2f
M2877 nw398 nw210 vdd vdd pch w=2u l=180n
M2878 nw398 nw104 vdd vdd pch w=2u l=180n
CT1042 t1042 0 0.1f
M2879 nw398 nw210 t1042 0 nch w=1u l=180n
M2880 t1042 nw104 0 0 nch w=1u l=180n
Cnw398 nw398 0 2f
M2881 nw399 nw211 0 0 nch w=1u l=180n
M2882 nw399 nw105 0 0 nch w=1u l=180n
CT1043 t1043 0 0.1f
M2883 t1043 nw211 vdd vdd pch w=2u l=180n
M2884 nw399 nw105 t1043 vdd pch w=2u l=180n
Cnw399 nw399 0 2f
CT1044 t1044 0 0.1f
M2885 t1044 nw212 vdd vdd pch w=2u l=180n
M2886 t1044 nw106 vdd vdd pch w=2u l=180n
CT1045 t1045 0 0.1f
M2887 t1044 nw212 t1045 0 nch w=1u l=180n
M2888 t1045 nw106 0 0 nch w=1u l=180n
M2889 nw400 t1044 vdd vdd pch w=2u l=180n
M2890 nw400 t1044 0 0 nch w=1u l=180n
Cnw400 nw400 0 2f
CT1046 t1046 0 0.1f
M2891 t1046 nw213 0 0 nch w=1u l=180n
M2892 t1046 nw107 0 0 nch w=1u l=180n
CT1047 t1047 0 0.1f
M2893 t1047 nw213 vdd vdd pch w=2u l=180n
M2894 t1046 nw107 t1047 vdd pch w=2u l=180n
M2895 nw401 t1046 vdd vdd pch w=2u l=180n
M2896 nw401 t1046 0 0 nch w=1u l=180n
Cnw401 nw401 0 2f
CT1048 t1048 0 0.1f
CT1049 t1049 0 0.1f
CT1050 t1050 0 0.1f
M2897 t1048 nw214 vdd vdd pch w=2u l=180n
M2898 t1048 nw108 vdd vdd pch w=2u l=180n
CT1051 t1051 0 0.1f
M2899 t1048 nw214 t1051 0 nch w=1u l=180n
M2900 t1051 nw108 0 0 nch w=1u l=180n
M2901 t1049 nw214 vdd vdd pch w=2u l=180n
M2902 t1049 t1048 vdd vdd pch w=2u l=180n
CT1052 t1052 0 0.1f
M2903 t1049 nw214 t1052 0 nch w=1u l=180n
M2904 t1052 t1048 0 0 nch w=1u l=180n
M2905 t1050 nw108 vdd vdd pch w=2u l=180n
M2906 t1050 t1048 vdd vdd pch w=2u l=180n
CT1053 t1053 0 0.1f
M2907 t1050 nw108 t1053 0 nch w=1u l=180n
M2908 t1053 t1048 0 0 nch w=1u l=180n
M2909 nw402 t1049 vdd vdd pch w=2u l=180n
M2910 nw402 t1050 vdd vdd pch w=2u l=180n
CT1054 t1054 0 0.1f
M2911 nw402 t1049 t1054 0 nch w=1u l=180n
M2912 t1054 t1050 0 0 nch w=1u l=180n
Cnw402 nw402 0 2f
M2913 nw403 nw215 vdd vdd pch w=2u l=180n
M2914 nw403 nw109 vdd vdd pch w=2u l=180n
CT1055 t1055 0 0.1f
M2915 nw403 nw215 t1055 0 nch w=1u l=180n
M2916 t1055 nw109 0 0 nch w=1u l=180n
Cnw403 nw403 0 2f
M2917 nw404 nw216 0 0 nch w=1u l=180n
M2918 nw404 nw110 0 0 nch w=1u l=180n
CT1056 t1056 0 0.1f
M2919 t1056 nw216 vdd vdd pch w=2u l=180n
M2920 nw404 nw110 t1056 vdd pch w=2u l=180n
Cnw404 nw404 0 2f
CT1057 t1057 0 0.1f
M2921 t1057 nw217 vdd vdd pch w=2u l=180n
M2922 t1057 nw111 vdd vdd pch w=2u l=180n
CT1058 t1058 0 0.1f
M2923 t1057 nw217 t1058 0 nch w=1u l=180n
M2924 t1058 nw111 0 0 nch w=1u l=180n
M2925 nw405 t1057 vdd vdd pch w=2u l=180n
M2926 nw405 t1057 0 0 nch w=1u l=180n
Cnw405 nw405 0 2f
CT1059 t1059 0 0.1f
M2927 t1059 nw218 0 0 nch w=1u l=180n
M2928 t1059 nw112 0 0 nch w=1u l=180n
CT1060 t1060 0 0.1f
M2929 t1060 nw218 vdd vdd pch w=2u l=180n
M2930 t1059 nw112 t1060 vdd pch w=2u l=180n
M2931 nw406 t1059 vdd vdd pch w=2u l=180n
M2932 nw406 t1059 0 0 nch w=1u l=180n
Cnw406 nw406 0 2f
CT1061 t1061 0 0.1f
CT1062 t1062 0 0.1f
CT1063 t1063 0 0.1f
M2933 t1061 nw219 vdd vdd pch w=2u l=180n
M2934 t1061 nw113 vdd vdd pch w=2u l=180n
CT1064 t1064 0 0.1f
M2935 t1061 nw219 t1064 0 nch w=1u l=180n
M2936 t1064 nw113 0 0 nch w=1u l=180n
M2937 t1062 nw219 vdd vdd pch w=2u l=180n
M2938 t1062 t1061 vdd vdd pch w=2u l=180n
CT1065 t1065 0 0.1f
M2939 t1062 nw219 t1065 0 nch w=1u l=180n
M2940 t1065 t1061 0 0 nch w=1u l=180n
M2941 t1063 nw113 vdd vdd pch w=2u l=180n
M2942 t1063 t1061 vdd vdd pch w=2u l=180n
CT1066 t1066 0 0.1f
M2943 t1063 nw113 t1066 0 nch w=1u l=180n
M2944 t1066 t1061 0 0 nch w=1u l=180n
M2945 nw407 t1062 vdd vdd pch w=2u l=180n
M2946 nw407 t1063 vdd vdd pch w=2u l=180n
CT1067 t1067 0 0.1f
M2947 nw407 t1062 t1067 0 nch w=1u l=180n
M2948 t1067 t1063 0 0 nch w=1u l=180n
Cnw407 nw407 0 2f
M2949 nw408 nw220 vdd vdd pch w=2u l=180n
M2950 nw408 nw114 vdd vdd pch w=2u l=180n
CT1068 t1068 0 0.1f
M2951 nw408 nw220 t1068 0 nch w=1u l=180n
M2952 t1068 nw114 0 0 nch w=1u l=180n
Cnw408 nw408 0 2f
M2953 nw409 nw221 0 0 nch w=1u l=180n
M2954 nw409 nw115 0 0 nch w=1u l=180n
CT1069 t1069 0 0.1f
M2955 t1069 nw221 vdd vdd pch w=2u l=180n
M2956 nw409 nw115 t1069 vdd pch w=2u l=180n
Cnw409 nw409 0 2f
CT1070 t1070 0 0.1f
M2957 t1070 nw222 vdd vdd pch w=2u l=180n
M2958 t1070 nw116 vdd vdd pch w=2u l=180n
CT1071 t1071 0 0.1f
M2959 t1070 nw222 t1071 0 nch w=1u l=180n
M2960 t1071 nw116 0 0 nch w=1u l=180n
M2961 nw410 t1070 vdd vdd pch w=2u l=180n
M2962 nw410 t1070 0 0 nch w=1u l=180n
Cnw410 nw410 0 2f
CT1072 t1072 0 0.1f
M2963 t1072 nw223 0 0 nch w=1u l=180n
M2964 t1072 nw117 0 0 nch w=1u l=180n
CT1073 t1073 0 0.1f
M2965 t1073 nw223 vdd vdd pch w=2u l=180n
M2966 t1072 nw117 t1073 vdd pch w=2u l=180n
M2967 nw411 t1072 vdd vdd pch w=2u l=180n
M2968 nw411 t1072 0 0 nch w=1u l=180n
Cnw411 nw411 0 2f
CT1074 t1074 0 0.1f
CT1075 t1075 0 0.1f
CT1076 t1076 0 0.1f
M2969 t1074 nw224 vdd vdd pch w=2u l=180n
M2970 t1074 nw118 vdd vdd pch w=2u l=180n
CT1077 t1077 0 0.1f
M2971 t1074 nw224 t1077 0 nch w=1u l=180n
M2972 t1077 nw118 0 0 nch w=1u l=180n
M2973 t1075 nw224 vdd vdd pch w=2u l=180n
M2974 t1075 t1074 vdd vdd pch w=2u l=180n
CT1078 t1078 0 0.1f
M2975 t1075 nw224 t1078 0 nch w=1u l=180n
M2976 t1078 t1074 0 0 nch w=1u l=180n
M2977 t1076 nw118 vdd vdd pch w=2u l=180n
M2978 t1076 t1074 vdd vdd pch w=2u l=180n
CT1079 t1079 0 0.1f
M2979 t1076 nw118 t1079 0 nch w=1u l=180n
M2980 t1079 t1074 0 0 nch w=1u l=180n
M2981 nw412 t1075 vdd vdd pch w=2u l=180n
M2982 nw412 t1076 vdd vdd pch w=2u l=180n
CT1080 t1080 0 0.1f
M2983 nw412 t1075 t1080 0 nch w=1u l=180n
M2984 t1080 t1076 0 0 nch w=1u l=180n
Cnw412 nw412 0 2f
M2985 nw413 nw225 vdd vdd pch w=2u l=180n
M2986 nw413 nw119 vdd vdd pch w=2u l=180n
CT1081 t1081 0 0.1f
M2987 nw413 nw225 t1081 0 nch w=1u l=180n
M2988 t1081 nw119 0 0 nch w=1u l=180n
Cnw413 nw413 0 2f
M2989 nw414 nw226 0 0 nch w=1u l=180n
M2990 nw414 nw120 0 0 nch w=1u l=180n
CT1082 t1082 0 0.1f
M2991 t1082 nw226 vdd vdd pch w=2u l=180n
M2992 nw414 nw120 t1082 vdd pch w=2u l=180n
Cnw414 nw414 0 2f
CT1083 t1083 0 0.1f
M2993 t1083 nw227 vdd vdd pch w=2u l=180n
M2994 t1083 nw121 vdd vdd pch w=2u l=180n
CT1084 t1084 0 0.1f
M2995 t1083 nw227 t1084 0 nch w=1u l=180n
M2996 t1084 nw121 0 0 nch w=1u l=180n
M2997 nw415 t1083 vdd vdd pch w=2u l=180n
M2998 nw415 t1083 0 0 nch w=1u l=180n
Cnw415 nw415 0 2f
CT1085 t1085 0 0.1f
M2999 t1085 nw228 0 0 nch w=1u l=180n
M3000 t1085 nw122 0 0 nch w=1u l=180n
CT1086 t1086 0 0.1f
M3001 t1086 nw228 vdd vdd pch w=2u l=180n
M3002 t1085 nw122 t1086 vdd pch w=2u l=180n
M3003 nw416 t1085 vdd vdd pch w=2u l=180n
M3004 nw416 t1085 0 0 nch w=1u l=180n
Cnw416 nw416 0 2f
CT1087 t1087 0 0.1f
CT1088 t1088 0 0.1f
CT1089 t1089 0 0.1f
M3005 t1087 nw229 vdd vdd pch w=2u l=180n
M3006 t1087 nw123 vdd vdd pch w=2u l=180n
CT1090 t1090 0 0.1f
M3007 t1087 nw229 t1090 0 nch w=1u l=180n
M3008 t1090 nw123 0 0 nch w=1u l=180n
M3009 t1088 nw229 vdd vdd pch w=2u l=180n
M3010 t1088 t1087 vdd vdd pch w=2u l=180n
CT1091 t1091 0 0.1f
M3011 t1088 nw229 t1091 0 nch w=1u l=180n
M3012 t1091 t1087 0 0 nch w=1u l=180n
M3013 t1089 nw123 vdd vdd pch w=2u l=180n
M3014 t1089 t1087 vdd vdd pch w=2u l=180n
CT1092 t1092 0 0.1f
M3015 t1089 nw123 t1092 0 nch w=1u l=180n
M3016 t1092 t1087 0 0 nch w=1u l=180n
M3017 nw417 t1088 vdd vdd pch w=2u l=180n
M3018 nw417 t1089 vdd vdd pch w=2u l=180n
CT1093 t1093 0 0.1f
M3019 nw417 t1088 t1093 0 nch w=1u l=180n
M3020 t1093 t1089 0 0 nch w=1u l=180n
Cnw417 nw417 0 2f
M3021 nw418 nw230 vdd vdd pch w=2u l=180n
M3022 nw418 nw124 vdd vdd pch w=2u l=180n
CT1094 t1094 0 0.1f
M3023 nw418 nw230 t1094 0 nch w=1u l=180n
M3024 t1094 nw124 0 0 nch w=1u l=180n
Cnw418 nw418 0 2f
M3025 nw419 nw231 0 0 nch w=1u l=180n
M3026 nw419 nw125 0 0 nch w=1u l=180n
CT1095 t1095 0 0.1f
M3027 t1095 nw231 vdd vdd pch w=2u l=180n
M3028 nw419 nw125 t1095 vdd pch w=2u l=180n
Cnw419 nw419 0 2f
CT1096 t1096 0 0.1f
M3029 t1096 nw232 vdd vdd pch w=2u l=180n
M3030 t1096 nw126 vdd vdd pch w=2u l=180n
CT1097 t1097 0 0.1f
M3031 t1096 nw232 t1097 0 nch w=1u l=180n
M3032 t1097 nw126 0 0 nch w=1u l=180n
M3033 nw420 t1096 vdd vdd pch w=2u l=180n
M3034 nw420 t1096 0 0 nch w=1u l=180n
Cnw420 nw420 0 2f
CT1098 t1098 0 0.1f
M3035 t1098 nw233 0 0 nch w=1u l=180n
M3036 t1098 nw127 0 0 nch w=1u l=180n
CT1099 t1099 0 0.1f
M3037 t1099 nw233 vdd vdd pch w=2u l=180n
M3038 t1098 nw127 t1099 vdd pch w=2u l=180n
M3039 nw421 t1098 vdd vdd pch w=2u l=180n
M3040 nw421 t1098 0 0 nch w=1u l=180n
Cnw421 nw421 0 2f
CT1100 t1100 0 0.1f
CT1101 t1101 0 0.1f
CT1102 t1102 0 0.1f
M3041 t1100 nw234 vdd vdd pch w=2u l=180n
M3042 t1100 nw128 vdd vdd pch w=2u l=180n
CT1103 t1103 0 0.1f
M3043 t1100 nw234 t1103 0 nch w=1u l=180n
M3044 t1103 nw128 0 0 nch w=1u l=180n
M3045 t1101 nw234 vdd vdd pch w=2u l=180n
M3046 t1101 t1100 vdd vdd pch w=2u l=180n
CT1104 t1104 0 0.1f
M3047 t1101 nw234 t1104 0 nch w=1u l=180n
M3048 t1104 t1100 0 0 nch w=1u l=180n
M3049 t1102 nw128 vdd vdd pch w=2u l=180n
M3050 t1102 t1100 vdd vdd pch w=2u l=180n
CT1105 t1105 0 0.1f
M3051 t1102 nw128 t1105 0 nch w=1u l=180n
M3052 t1105 t1100 0 0 nch w=1u l=180n
M3053 nw422 t1101 vdd vdd pch w=2u l=180n
M3054 nw422 t1102 vdd vdd pch w=2u l=180n
CT1106 t1106 0 0.1f
M3055 nw422 t1101 t1106 0 nch w=1u l=180n
M3056 t1106 t1102 0 0 nch w=1u l=180n
Cnw422 nw422 0 2f
M3057 nw423 nw235 vdd vdd pch w=2u l=180n
M3058 nw423 nw129 vdd vdd pch w=2u l=180n
CT1107 t1107 0 0.1f
M3059 nw423 nw235 t1107 0 nch w=1u l=180n
M3060 t1107 nw129 0 0 nch w=1u l=180n
Cnw423 nw423 0 2f
M3061 nw424 nw236 0 0 nch w=1u l=180n
M3062 nw424 nw130 0 0 nch w=1u l=180n
CT1108 t1108 0 0.1f
M3063 t1108 nw236 vdd vdd pch w=2u l=180n
M3064 nw424 nw130 t1108 vdd pch w=2u l=180n
Cnw424 nw424 0 2f
CT1109 t1109 0 0.1f
M3065 t1109 nw237 vdd vdd pch w=2u l=180n
M3066 t1109 nw131 vdd vdd pch w=2u l=180n
CT1110 t1110 0 0.1f
M3067 t1109 nw237 t1110 0 nch w=1u l=180n
M3068 t1110 nw131 0 0 nch w=1u l=180n
M3069 nw425 t1109 vdd vdd pch w=2u l=180n
M3070 nw425 t1109 0 0 nch w=1u l=180n
Cnw425 nw425 0 2f
CT1111 t1111 0 0.1f
M3071 t1111 nw238 0 0 nch w=1u l=180n
M3072 t1111 nw132 0 0 nch w=1u l=180n
CT1112 t1112 0 0.1f
M3073 t1112 nw238 vdd vdd pch w=2u l=180n
M3074 t1111 nw132 t1112 vdd pch w=2u l=180n
M3075 nw426 t1111 vdd vdd pch w=2u l=180n
M3076 nw426 t1111 0 0 nch w=1u l=180n
Cnw426 nw426 0 2f
CT1113 t1113 0 0.1f
CT1114 t1114 0 0.1f
CT1115 t1115 0 0.1f
M3077 t1113 nw239 vdd vdd pch w=2u l=180n
M3078 t1113 nw133 vdd vdd pch w=2u l=180n
CT1116 t1116 0 0.1f
M3079 t1113 nw239 t1116 0 nch w=1u l=180n
M3080 t1116 nw133 0 0 nch w=1u l=180n
M3081 t1114 nw239 vdd vdd pch w=2u l=180n
M3082 t1114 t1113 vdd vdd pch w=2u l=180n
CT1117 t1117 0 0.1f
M3083 t1114 nw239 t1117 0 nch w=1u l=180n
M3084 t1117 t1113 0 0 nch w=1u l=180n
M3085 t1115 nw133 vdd vdd pch w=2u l=180n
M3086 t1115 t1113 vdd vdd pch w=2u l=180n
CT1118 t1118 0 0.1f
M3087 t1115 nw133 t1118 0 nch w=1u l=180n
M3088 t1118 t1113 0 0 nch w=1u l=180n
M3089 nw427 t1114 vdd vdd pch w=2u l=180n
M3090 nw427 t1115 vdd vdd pch w=2u l=180n
CT1119 t1119 0 0.1f
M3091 nw427 t1114 t1119 0 nch w=1u l=180n
M3092 t1119 t1115 0 0 nch w=1u l=180n
Cnw427 nw427 0 2f
M3093 nw428 nw240 vdd vdd pch w=2u l=180n
M3094 nw428 nw134 vdd vdd pch w=2u l=180n
CT1120 t1120 0 0.1f
M3095 nw428 nw240 t1120 0 nch w=1u l=180n
M3096 t1120 nw134 0 0 nch w=1u l=180n
Cnw428 nw428 0 2f
M3097 nw429 nw241 0 0 nch w=1u l=180n
M3098 nw429 nw135 0 0 nch w=1u l=180n
CT1121 t1121 0 0.1f
M3099 t1121 nw241 vdd vdd pch w=2u l=180n
M3100 nw429 nw135 t1121 vdd pch w=2u l=180n
Cnw429 nw429 0 2f
CT1122 t1122 0 0.1f
M3101 t1122 nw242 vdd vdd pch w=2u l=180n
M3102 t1122 nw136 vdd vdd pch w=2u l=180n
CT1123 t1123 0 0.1f
M3103 t1122 nw242 t1123 0 nch w=1u l=180n
M3104 t1123 nw136 0 0 nch w=1u l=180n
M3105 nw430 t1122 vdd vdd pch w=2u l=180n
M3106 nw430 t1122 0 0 nch w=1u l=180n
Cnw430 nw430 0 2f
CT1124 t1124 0 0.1f
M3107 t1124 nw243 0 0 nch w=1u l=180n
M3108 t1124 nw137 0 0 nch w=1u l=180n
CT1125 t1125 0 0.1f
M3109 t1125 nw243 vdd vdd pch w=2u l=180n
M3110 t1124 nw137 t1125 vdd pch w=2u l=180n
M3111 nw431 t1124 vdd vdd pch w=2u l=180n
M3112 nw431 t1124 0 0 nch w=1u l=180n
Cnw431 nw431 0 2f
CT1126 t1126 0 0.1f
CT1127 t1127 0 0.1f
CT1128 t1128 0 0.1f
M3113 t1126 nw244 vdd vdd pch w=2u l=180n
M3114 t1126 nw138 vdd vdd pch w=2u l=180n
CT1129 t1129 0 0.1f
M3115 t1126 nw244 t1129 0 nch w=1u l=180n
M3116 t1129 nw138 0 0 nch w=1u l=180n
M3117 t1127 nw244 vdd vdd pch w=2u l=180n
M3118 t1127 t1126 vdd vdd pch w=2u l=180n
CT1130 t1130 0 0.1f
M3119 t1127 nw244 t1130 0 nch w=1u l=180n
M3120 t1130 t1126 0 0 nch w=1u l=180n
M3121 t1128 nw138 vdd vdd pch w=2u l=180n
M3122 t1128 t1126 vdd vdd pch w=2u l=180n
CT1131 t1131 0 0.1f
M3123 t1128 nw138 t1131 0 nch w=1u l=180n
M3124 t1131 t1126 0 0 nch w=1u l=180n
M3125 nw432 t1127 vdd vdd pch w=2u l=180n
M3126 nw432 t1128 vdd vdd pch w=2u l=180n
CT1132 t1132 0 0.1f
M3127 nw432 t1127 t1132 0 nch w=1u l=180n
M3128 t1132 t1128 0 0 nch w=1u l=180n
Cnw432 nw432 0 2f
M3129 nw433 nw245 vdd vdd pch w=2u l=180n
M3130 nw433 nw139 vdd vdd pch w=2u l=180n
CT1133 t1133 0 0.1f
M3131 nw433 nw245 t1133 0 nch w=1u l=180n
M3132 t1133 nw139 0 0 nch w=1u l=180n
Cnw433 nw433 0 2f
M3133 nw434 nw246 0 0 nch w=1u l=180n
M3134 nw434 nw140 0 0 nch w=1u l=180n
CT1134 t1134 0 0.1f
M3135 t1134 nw246 vdd vdd pch w=2u l=180n
M3136 nw434 nw140 t1134 vdd pch w=2u l=180n
Cnw434 nw434 0 2f
CT1135 t1135 0 0.1f
M3137 t1135 nw247 vdd vdd pch w=2u l=180n
M3138 t1135 nw141 vdd vdd pch w=2u l=180n
CT1136 t1136 0 0.1f
M3139 t1135 nw247 t1136 0 nch w=1u l=180n
M3140 t1136 nw141 0 0 nch w=1u l=180n
M3141 nw435 t1135 vdd vdd pch w=2u l=180n
M3142 nw435 t1135 0 0 nch w=1u l=180n
Cnw435 nw435 0 2f
CT1137 t1137 0 0.1f
M3143 t1137 nw248 0 0 nch w=1u l=180n
M3144 t1137 nw142 0 0 nch w=1u l=180n
CT1138 t1138 0 0.1f
M3145 t1138 nw248 vdd vdd pch w=2u l=180n
M3146 t1137 nw142 t1138 vdd pch w=2u l=180n
M3147 nw436 t1137 vdd vdd pch w=2u l=180n
M3148 nw436 t1137 0 0 nch w=1u l=180n
Cnw436 nw436 0 2f
CT1139 t1139 0 0.1f
CT1140 t1140 0 0.1f
CT1141 t1141 0 0.1f
M3149 t1139 nw249 vdd vdd pch w=2u l=180n
M3150 t1139 nw143 vdd vdd pch w=2u l=180n
CT1142 t1142 0 0.1f
M3151 t1139 nw249 t1142 0 nch w=1u l=180n
M3152 t1142 nw143 0 0 nch w=1u l=180n
M3153 t1140 nw249 vdd vdd pch w=2u l=180n
M3154 t1140 t1139 vdd vdd pch w=2u l=180n
CT1143 t1143 0 0.1f
M3155 t1140 nw249 t1143 0 nch w=1u l=180n
M3156 t1143 t1139 0 0 nch w=1u l=180n
M3157 t1141 nw143 vdd vdd pch w=2u l=180n
M3158 t1141 t1139 vdd vdd pch w=2u l=180n
CT1144 t1144 0 0.1f
M3159 t1141 nw143 t1144 0 nch w=1u l=180n
M3160 t1144 t1139 0 0 nch w=1u l=180n
M3161 nw437 t1140 vdd vdd pch w=2u l=180n
M3162 nw437 t1141 vdd vdd pch w=2u l=180n
CT1145 t1145 0 0.1f
M3163 nw437 t1140 t1145 0 nch w=1u l=180n
M3164 t1145 t1141 0 0 nch w=1u l=180n
Cnw437 nw437 0 2f
M3165 nw438 nw250 vdd vdd pch w=2u l=180n
M3166 nw438 nw144 vdd vdd pch w=2u l=180n
CT1146 t1146 0 0.1f
M3167 nw438 nw250 t1146 0 nch w=1u l=180n
M3168 t1146 nw144 0 0 nch w=1u l=180n
Cnw438 nw438 0 2f
M3169 nw439 nw251 0 0 nch w=1u l=180n
M3170 nw439 nw145 0 0 nch w=1u l=180n
CT1147 t1147 0 0.1f
M3171 t1147 nw251 vdd vdd pch w=2u l=180n
M3172 nw439 nw145 t1147 vdd pch w=2u l=180n
Cnw439 nw439 0 2f
CT1148 t1148 0 0.1f
M3173 t1148 nw252 vdd vdd pch w=2u l=180n
M3174 t1148 nw146 vdd vdd pch w=2u l=180n
CT1149 t1149 0 0.1f
M3175 t1148 nw252 t1149 0 nch w=1u l=180n
M3176 t1149 nw146 0 0 nch w=1u l=180n
M3177 nw440 t1148 vdd vdd pch w=2u l=180n
M3178 nw440 t1148 0 0 nch w=1u l=180n
Cnw440 nw440 0 2f
CT1150 t1150 0 0.1f
M3179 t1150 nw253 0 0 nch w=1u l=180n
M3180 t1150 nw147 0 0 nch w=1u l=180n
CT1151 t1151 0 0.1f
M3181 t1151 nw253 vdd vdd pch w=2u l=180n
M3182 t1150 nw147 t1151 vdd pch w=2u l=180n
M3183 nw441 t1150 vdd vdd pch w=2u l=180n
M3184 nw441 t1150 0 0 nch w=1u l=180n
Cnw441 nw441 0 2f
CT1152 t1152 0 0.1f
CT1153 t1153 0 0.1f
CT1154 t1154 0 0.1f
M3185 t1152 nw254 vdd vdd pch w=2u l=180n
M3186 t1152 nw148 vdd vdd pch w=2u l=180n
CT1155 t1155 0 0.1f
M3187 t1152 nw254 t1155 0 nch w=1u l=180n
M3188 t1155 nw148 0 0 nch w=1u l=180n
M3189 t1153 nw254 vdd vdd pch w=2u l=180n
M3190 t1153 t1152 vdd vdd pch w=2u l=180n
CT1156 t1156 0 0.1f
M3191 t1153 nw254 t1156 0 nch w=1u l=180n
M3192 t1156 t1152 0 0 nch w=1u l=180n
M3193 t1154 nw148 vdd vdd pch w=2u l=180n
M3194 t1154 t1152 vdd vdd pch w=2u l=180n
CT1157 t1157 0 0.1f
M3195 t1154 nw148 t1157 0 nch w=1u l=180n
M3196 t1157 t1152 0 0 nch w=1u l=180n
M3197 nw442 t1153 vdd vdd pch w=2u l=180n
M3198 nw442 t1154 vdd vdd pch w=2u l=180n
CT1158 t1158 0 0.1f
M3199 nw442 t1153 t1158 0 nch w=1u l=180n
M3200 t1158 t1154 0 0 nch w=1u l=180n
Cnw442 nw442 0 2f
M3201 nw443 nw255 vdd vdd pch w=2u l=180n
M3202 nw443 nw149 vdd vdd pch w=2u l=180n
CT1159 t1159 0 0.1f
M3203 nw443 nw255 t1159 0 nch w=1u l=180n
M3204 t1159 nw149 0 0 nch w=1u l=180n
Cnw443 nw443 0 2f
M3205 nw444 nw256 0 0 nch w=1u l=180n
M3206 nw444 nw150 0 0 nch w=1u l=180n
CT1160 t1160 0 0.1f
M3207 t1160 nw256 vdd vdd pch w=2u l=180n
M3208 nw444 nw150 t1160 vdd pch w=2u l=180n
Cnw444 nw444 0 2f
CT1161 t1161 0 0.1f
M3209 t1161 nw257 vdd vdd pch w=2u l=180n
M3210 t1161 nw151 vdd vdd pch w=2u l=180n
CT1162 t1162 0 0.1f
M3211 t1161 nw257 t1162 0 nch w=1u l=180n
M3212 t1162 nw151 0 0 nch w=1u l=180n
M3213 nw445 t1161 vdd vdd pch w=2u l=180n
M3214 nw445 t1161 0 0 nch w=1u l=180n
Cnw445 nw445 0 2f
CT1163 t1163 0 0.1f
M3215 t1163 nw258 0 0 nch w=1u l=180n
M3216 t1163 nw152 0 0 nch w=1u l=180n
CT1164 t1164 0 0.1f
M3217 t1164 nw258 vdd vdd pch w=2u l=180n
M3218 t1163 nw152 t1164 vdd pch w=2u l=180n
M3219 nw446 t1163 vdd vdd pch w=2u l=180n
M3220 nw446 t1163 0 0 nch w=1u l=180n
Cnw446 nw446 0 2f
CT1165 t1165 0 0.1f
CT1166 t1166 0 0.1f
CT1167 t1167 0 0.1f
M3221 t1165 nw259 vdd vdd pch w=2u l=180n
M3222 t1165 nw153 vdd vdd pch w=2u l=180n
CT1168 t1168 0 0.1f
M3223 t1165 nw259 t1168 0 nch w=1u l=180n
M3224 t1168 nw153 0 0 nch w=1u l=180n
M3225 t1166 nw259 vdd vdd pch w=2u l=180n
M3226 t1166 t1165 vdd vdd pch w=2u l=180n
CT1169 t1169 0 0.1f
M3227 t1166 nw259 t1169 0 nch w=1u l=180n
M3228 t1169 t1165 0 0 nch w=1u l=180n
M3229 t1167 nw153 vdd vdd pch w=2u l=180n
M3230 t1167 t1165 vdd vdd pch w=2u l=180n
CT1170 t1170 0 0.1f
M3231 t1167 nw153 t1170 0 nch w=1u l=180n
M3232 t1170 t1165 0 0 nch w=1u l=180n
M3233 nw447 t1166 vdd vdd pch w=2u l=180n
M3234 nw447 t1167 vdd vdd pch w=2u l=180n
CT1171 t1171 0 0.1f
M3235 nw447 t1166 t1171 0 nch w=1u l=180n
M3236 t1171 t1167 0 0 nch w=1u l=180n
Cnw447 nw447 0 2f
M3237 nw448 nw260 vdd vdd pch w=2u l=180n
M3238 nw448 nw154 vdd vdd pch w=2u l=180n
CT1172 t1172 0 0.1f
M3239 nw448 nw260 t1172 0 nch w=1u l=180n
M3240 t1172 nw154 0 0 nch w=1u l=180n
Cnw448 nw448 0 2f
M3241 nw449 nw261 0 0 nch w=1u l=180n
M3242 nw449 nw155 0 0 nch w=1u l=180n
CT1173 t1173 0 0.1f
M3243 t1173 nw261 vdd vdd pch w=2u l=180n
M3244 nw449 nw155 t1173 vdd pch w=2u l=180n
Cnw449 nw449 0 2f
CT1174 t1174 0 0.1f
M3245 t1174 nw262 vdd vdd pch w=2u l=180n
M3246 t1174 nw156 vdd vdd pch w=2u l=180n
CT1175 t1175 0 0.1f
M3247 t1174 nw262 t1175 0 nch w=1u l=180n
M3248 t1175 nw156 0 0 nch w=1u l=180n
M3249 nw450 t1174 vdd vdd pch w=2u l=180n
M3250 nw450 t1174 0 0 nch w=1u l=180n
Cnw450 nw450 0 2f
CT1176 t1176 0 0.1f
M3251 t1176 nw263 0 0 nch w=1u l=180n
M3252 t1176 nw157 0 0 nch w=1u l=180n
CT1177 t1177 0 0.1f
M3253 t1177 nw263 vdd vdd pch w=2u l=180n
M3254 t1176 nw157 t1177 vdd pch w=2u l=180n
M3255 nw451 t1176 vdd vdd pch w=2u l=180n
M3256 nw451 t1176 0 0 nch w=1u l=180n
Cnw451 nw451 0 2f
CT1178 t1178 0 0.1f
CT1179 t1179 0 0.1f
CT1180 t1180 0 0.1f
M3257 t1178 nw264 vdd vdd pch w=2u l=180n
M3258 t1178 nw158 vdd vdd pch w=2u l=180n
CT1181 t1181 0 0.1f
M3259 t1178 nw264 t1181 0 nch w=1u l=180n
M3260 t1181 nw158 0 0 nch w=1u l=180n
M3261 t1179 nw264 vdd vdd pch w=2u l=180n
M3262 t1179 t1178 vdd vdd pch w=2u l=180n
CT1182 t1182 0 0.1f
M3263 t1179 nw264 t1182 0 nch w=1u l=180n
M3264 t1182 t1178 0 0 nch w=1u l=180n
M3265 t1180 nw158 vdd vdd pch w=2u l=180n
M3266 t1180 t1178 vdd vdd pch w=2u l=180n
CT1183 t1183 0 0.1f
M3267 t1180 nw158 t1183 0 nch w=1u l=180n
M3268 t1183 t1178 0 0 nch w=1u l=180n
M3269 nw452 t1179 vdd vdd pch w=2u l=180n
M3270 nw452 t1180 vdd vdd pch w=2u l=180n
CT1184 t1184 0 0.1f
M3271 nw452 t1179 t1184 0 nch w=1u l=180n
M3272 t1184 t1180 0 0 nch w=1u l=180n
Cnw452 nw452 0 2f
M3273 nw453 nw265 vdd vdd pch w=2u l=180n
M3274 nw453 nw159 vdd vdd pch w=2u l=180n
CT1185 t1185 0 0.1f
M3275 nw453 nw265 t1185 0 nch w=1u l=180n
M3276 t1185 nw159 0 0 nch w=1u l=180n
Cnw453 nw453 0 2f
M3277 nw454 nw266 0 0 nch w=1u l=180n
M3278 nw454 nw160 0 0 nch w=1u l=180n
CT1186 t1186 0 0.1f
M3279 t1186 nw266 vdd vdd pch w=2u l=180n
M3280 nw454 nw160 t1186 vdd pch w=2u l=180n
Cnw454 nw454 0 2f
CT1187 t1187 0 0.1f
M3281 t1187 nw267 vdd vdd pch w=2u l=180n
M3282 t1187 nw161 vdd vdd pch w=2u l=180n
CT1188 t1188 0 0.1f
M3283 t1187 nw267 t1188 0 nch w=1u l=180n
M3284 t1188 nw161 0 0 nch w=1u l=180n
M3285 nw455 t1187 vdd vdd pch w=2u l=180n
M3286 nw455 t1187 0 0 nch w=1u l=180n
Cnw455 nw455 0 2f
CT1189 t1189 0 0.1f
M3287 t1189 nw268 0 0 nch w=1u l=180n
M3288 t1189 nw162 0 0 nch w=1u l=180n
CT1190 t1190 0 0.1f
M3289 t1190 nw268 vdd vdd pch w=2u l=180n
M3290 t1189 nw162 t1190 vdd pch w=2u l=180n
M3291 nw456 t1189 vdd vdd pch w=2u l=180n
M3292 nw456 t1189 0 0 nch w=1u l=180n
Cnw456 nw456 0 2f
CT1191 t1191 0 0.1f
CT1192 t1192 0 0.1f
CT1193 t1193 0 0.1f
M3293 t1191 nw269 vdd vdd pch w=2u l=180n
M3294 t1191 nw163 vdd vdd pch w=2u l=180n
CT1194 t1194 0 0.1f
M3295 t1191 nw269 t1194 0 nch w=1u l=180n
M3296 t1194 nw163 0 0 nch w=1u l=180n
M3297 t1192 nw269 vdd vdd pch w=2u l=180n
M3298 t1192 t1191 vdd vdd pch w=2u l=180n
CT1195 t1195 0 0.1f
M3299 t1192 nw269 t1195 0 nch w=1u l=180n
M3300 t1195 t1191 0 0 nch w=1u l=180n
M3301 t1193 nw163 vdd vdd pch w=2u l=180n
M3302 t1193 t1191 vdd vdd pch w=2u l=180n
CT1196 t1196 0 0.1f
M3303 t1193 nw163 t1196 0 nch w=1u l=180n
M3304 t1196 t1191 0 0 nch w=1u l=180n
M3305 nw457 t1192 vdd vdd pch w=2u l=180n
M3306 nw457 t1193 vdd vdd pch w=2u l=180n
CT1197 t1197 0 0.1f
M3307 nw457 t1192 t1197 0 nch w=1u l=180n
M3308 t1197 t1193 0 0 nch w=1u l=180n
Cnw457 nw457 0 2f
M3309 nw458 nw270 vdd vdd pch w=2u l=180n
M3310 nw458 nw164 vdd vdd pch w=2u l=180n
CT1198 t1198 0 0.1f
M3311 nw458 nw270 t1198 0 nch w=1u l=180n
M3312 t1198 nw164 0 0 nch w=1u l=180n
Cnw458 nw458 0 2f
M3313 nw459 nw271 0 0 nch w=1u l=180n
M3314 nw459 nw165 0 0 nch w=1u l=180n
CT1199 t1199 0 0.1f
M3315 t1199 nw271 vdd vdd pch w=2u l=180n
M3316 nw459 nw165 t1199 vdd pch w=2u l=180n
Cnw459 nw459 0 2f
CT1200 t1200 0 0.1f
M3317 t1200 nw272 vdd vdd pch w=2u l=180n
M3318 t1200 nw166 vdd vdd pch w=2u l=180n
CT1201 t1201 0 0.1f
M3319 t1200 nw272 t1201 0 nch w=1u l=180n
M3320 t1201 nw166 0 0 nch w=1u l=180n
M3321 nw460 t1200 vdd vdd pch w=2u l=180n
M3322 nw460 t1200 0 0 nch w=1u l=180n
Cnw460 nw460 0 2f
CT1202 t1202 0 0.1f
M3323 t1202 nw273 0 0 nch w=1u l=180n
M3324 t1202 nw167 0 0 nch w=1u l=180n
CT1203 t1203 0 0.1f
M3325 t1203 nw273 vdd vdd pch w=2u l=180n
M3326 t1202 nw167 t1203 vdd pch w=2u l=180n
M3327 nw461 t1202 vdd vdd pch w=2u l=180n
M3328 nw461 t1202 0 0 nch w=1u l=180n
Cnw461 nw461 0 2f
CT1204 t1204 0 0.1f
CT1205 t1205 0 0.1f
CT1206 t1206 0 0.1f
M3329 t1204 nw274 vdd vdd pch w=2u l=180n
M3330 t1204 nw168 vdd vdd pch w=2u l=180n
CT1207 t1207 0 0.1f
M3331 t1204 nw274 t1207 0 nch w=1u l=180n
M3332 t1207 nw168 0 0 nch w=1u l=180n
M3333 t1205 nw274 vdd vdd pch w=2u l=180n
M3334 t1205 t1204 vdd vdd pch w=2u l=180n
CT1208 t1208 0 0.1f
M3335 t1205 nw274 t1208 0 nch w=1u l=180n
M3336 t1208 t1204 0 0 nch w=1u l=180n
M3337 t1206 nw168 vdd vdd pch w=2u l=180n
M3338 t1206 t1204 vdd vdd pch w=2u l=180n
CT1209 t1209 0 0.1f
M3339 t1206 nw168 t1209 0 nch w=1u l=180n
M3340 t1209 t1204 0 0 nch w=1u l=180n
M3341 nw462 t1205 vdd vdd pch w=2u l=180n
M3342 nw462 t1206 vdd vdd pch w=2u l=180n
CT1210 t1210 0 0.1f
M3343 nw462 t1205 t1210 0 nch w=1u l=180n
M3344 t1210 t1206 0 0 nch w=1u l=180n
Cnw462 nw462 0 2f
M3345 nw463 nw275 vdd vdd pch w=2u l=180n
M3346 nw463 nw169 vdd vdd pch w=2u l=180n
CT1211 t1211 0 0.1f
M3347 nw463 nw275 t1211 0 nch w=1u l=180n
M3348 t1211 nw169 0 0 nch w=1u l=180n
Cnw463 nw463 0 2f
M3349 nw464 nw276 0 0 nch w=1u l=180n
M3350 nw464 nw170 0 0 nch w=1u l=180n
CT1212 t1212 0 0.1f
M3351 t1212 nw276 vdd vdd pch w=2u l=180n
M3352 nw464 nw170 t1212 vdd pch w=2u l=180n
Cnw464 nw464 0 2f
CT1213 t1213 0 0.1f
M3353 t1213 nw277 vdd vdd pch w=2u l=180n
M3354 t1213 nw171 vdd vdd pch w=2u l=180n
CT1214 t1214 0 0.1f
M3355 t1213 nw277 t1214 0 nch w=1u l=180n
M3356 t1214 nw171 0 0 nch w=1u l=180n
M3357 nw465 t1213 vdd vdd pch w=2u l=180n
M3358 nw465 t1213 0 0 nch w=1u l=180n
Cnw465 nw465 0 2f
CT1215 t1215 0 0.1f
M3359 t1215 nw278 0 0 nch w=1u l=180n
M3360 t1215 nw172 0 0 nch w=1u l=180n
CT1216 t1216 0 0.1f
M3361 t1216 nw278 vdd vdd pch w=2u l=180n
M3362 t1215 nw172 t1216 vdd pch w=2u l=180n
M3363 nw466 t1215 vdd vdd pch w=2u l=180n
M3364 nw466 t1215 0 0 nch w=1u l=180n
Cnw466 nw466 0 2f
CT1217 t1217 0 0.1f
CT1218 t1218 0 0.1f
CT1219 t1219 0 0.1f
M3365 t1217 nw279 vdd vdd pch w=2u l=180n
M3366 t1217 nw173 vdd vdd pch w=2u l=180n
CT1220 t1220 0 0.1f
M3367 t1217 nw279 t1220 0 nch w=1u l=180n
M3368 t1220 nw173 0 0 nch w=1u l=180n
M3369 t1218 nw279 vdd vdd pch w=2u l=180n
M3370 t1218 t1217 vdd vdd pch w=2u l=180n
CT1221 t1221 0 0.1f
M3371 t1218 nw279 t1221 0 nch w=1u l=180n
M3372 t1221 t1217 0 0 nch w=1u l=180n
M3373 t1219 nw173 vdd vdd pch w=2u l=180n
M3374 t1219 t1217 vdd vdd pch w=2u l=180n
CT1222 t1222 0 0.1f
M3375 t1219 nw173 t1222 0 nch w=1u l=180n
M3376 t1222 t1217 0 0 nch w=1u l=180n
M3377 nw467 t1218 vdd vdd pch w=2u l=180n
M3378 nw467 t1219 vdd vdd pch w=2u l=180n
CT1223 t1223 0 0.1f
M3379 nw467 t1218 t1223 0 nch w=1u l=180n
M3380 t1223 t1219 0 0 nch w=1u l=180n
Cnw467 nw467 0 2f
M3381 nw468 nw280 vdd vdd pch w=2u l=180n
M3382 nw468 nw174 vdd vdd pch w=2u l=180n
CT1224 t1224 0 0.1f
M3383 nw468 nw280 t1224 0 nch w=1u l=180n
M3384 t1224 nw174 0 0 nch w=1u l=180n
Cnw468 nw468 0 2f
M3385 nw469 nw281 0 0 nch w=1u l=180n
M3386 nw469 nw175 0 0 nch w=1u l=180n
CT1225 t1225 0 0.1f
M3387 t1225 nw281 vdd vdd pch w=2u l=180n
M3388 nw469 nw175 t1225 vdd pch w=2u l=180n
Cnw469 nw469 0 2f
CT1226 t1226 0 0.1f
M3389 t1226 nw282 vdd vdd pch w=2u l=180n
M3390 t1226 nw176 vdd vdd pch w=2u l=180n
CT1227 t1227 0 0.1f
M3391 t1226 nw282 t1227 0 nch w=1u l=180n
M3392 t1227 nw176 0 0 nch w=1u l=180n
M3393 nw470 t1226 vdd vdd pch w=2u l=180n
M3394 nw470 t1226 0 0 nch w=1u l=180n
Cnw470 nw470 0 2f
CT1228 t1228 0 0.1f
M3395 t1228 nw283 0 0 nch w=1u l=180n
M3396 t1228 nw177 0 0 nch w=1u l=180n
CT1229 t1229 0 0.1f
M3397 t1229 nw283 vdd vdd pch w=2u l=180n
M3398 t1228 nw177 t1229 vdd pch w=2u l=180n
M3399 nw471 t1228 vdd vdd pch w=2u l=180n
M3400 nw471 t1228 0 0 nch w=1u l=180n
Cnw471 nw471 0 2f
CT1230 t1230 0 0.1f
CT1231 t1231 0 0.1f
CT1232 t1232 0 0.1f
M3401 t1230 nw284 vdd vdd pch w=2u l=180n
M3402 t1230 nw178 vdd vdd pch w=2u l=180n
CT1233 t1233 0 0.1f
M3403 t1230 nw284 t1233 0 nch w=1u l=180n
M3404 t1233 nw178 0 0 nch w=1u l=180n
M3405 t1231 nw284 vdd vdd pch w=2u l=180n
M3406 t1231 t1230 vdd vdd pch w=2u l=180n
CT1234 t1234 0 0.1f
M3407 t1231 nw284 t1234 0 nch w=1u l=180n
M3408 t1234 t1230 0 0 nch w=1u l=180n
M3409 t1232 nw178 vdd vdd pch w=2u l=180n
M3410 t1232 t1230 vdd vdd pch w=2u l=180n
CT1235 t1235 0 0.1f
M3411 t1232 nw178 t1235 0 nch w=1u l=180n
M3412 t1235 t1230 0 0 nch w=1u l=180n
M3413 nw472 t1231 vdd vdd pch w=2u l=180n
M3414 nw472 t1232 vdd vdd pch w=2u l=180n
CT1236 t1236 0 0.1f
M3415 nw472 t1231 t1236 0 nch w=1u l=180n
M3416 t1236 t1232 0 0 nch w=1u l=180n
Cnw472 nw472 0 2f
M3417 nw473 nw285 vdd vdd pch w=2u l=180n
M3418 nw473 nw179 vdd vdd pch w=2u l=180n
CT1237 t1237 0 0.1f
M3419 nw473 nw285 t1237 0 nch w=1u l=180n
M3420 t1237 nw179 0 0 nch w=1u l=180n
Cnw473 nw473 0 2f
M3421 nw474 nw286 0 0 nch w=1u l=180n
M3422 nw474 nw180 0 0 nch w=1u l=180n
CT1238 t1238 0 0.1f
M3423 t1238 nw286 vdd vdd pch w=2u l=180n
M3424 nw474 nw180 t1238 vdd pch w=2u l=180n
Cnw474 nw474 0 2f
CT1239 t1239 0 0.1f
M3425 t1239 nw287 vdd vdd pch w=2u l=180n
M3426 t1239 nw181 vdd vdd pch w=2u l=180n
CT1240 t1240 0 0.1f
M3427 t1239 nw287 t1240 0 nch w=1u l=180n
M3428 t1240 nw181 0 0 nch w=1u l=180n
M3429 nw475 t1239 vdd vdd pch w=2u l=180n
M3430 nw475 t1239 0 0 nch w=1u l=180n
Cnw475 nw475 0 2f
CT1241 t1241 0 0.1f
M3431 t1241 nw288 0 0 nch w=1u l=180n
M3432 t1241 nw182 0 0 nch w=1u l=180n
CT1242 t1242 0 0.1f
M3433 t1242 nw288 vdd vdd pch w=2u l=180n
M3434 t1241 nw182 t1242 vdd pch w=2u l=180n
M3435 nw476 t1241 vdd vdd pch w=2u l=180n
M3436 nw476 t1241 0 0 nch w=1u l=180n
Cnw476 nw476 0 2f
CT1243 t1243 0 0.1f
CT1244 t1244 0 0.1f
CT1245 t1245 0 0.1f
M3437 t1243 nw289 vdd vdd pch w=2u l=180n
M3438 t1243 nw183 vdd vdd pch w=2u l=180n
CT1246 t1246 0 0.1f
M3439 t1243 nw289 t1246 0 nch w=1u l=180n
M3440 t1246 nw183 0 0 nch w=1u l=180n
M3441 t1244 nw289 vdd vdd pch w=2u l=180n
M3442 t1244 t1243 vdd vdd pch w=2u l=180n
CT1247 t1247 0 0.1f
M3443 t1244 nw289 t1247 0 nch w=1u l=180n
M3444 t1247 t1243 0 0 nch w=1u l=180n
M3445 t1245 nw183 vdd vdd pch w=2u l=180n
M3446 t1245 t1243 vdd vdd pch w=2u l=180n
CT1248 t1248 0 0.1f
M3447 t1245 nw183 t1248 0 nch w=1u l=180n
M3448 t1248 t1243 0 0 nch w=1u l=180n
M3449 nw477 t1244 vdd vdd pch w=2u l=180n
M3450 nw477 t1245 vdd vdd pch w=2u l=180n
CT1249 t1249 0 0.1f
M3451 nw477 t1244 t1249 0 nch w=1u l=180n
M3452 t1249 t1245 0 0 nch w=1u l=180n
Cnw477 nw477 0 2f
M3453 nw478 nw290 vdd vdd pch w=2u l=180n
M3454 nw478 nw184 vdd vdd pch w=2u l=180n
CT1250 t1250 0 0.1f
M3455 nw478 nw290 t1250 0 nch w=1u l=180n
M3456 t1250 nw184 0 0 nch w=1u l=180n
Cnw478 nw478 0 2f
M3457 nw479 nw291 0 0 nch w=1u l=180n
M3458 nw479 nw185 0 0 nch w=1u l=180n
CT1251 t1251 0 0.1f
M3459 t1251 nw291 vdd vdd pch w=2u l=180n
M3460 nw479 nw185 t1251 vdd pch w=2u l=180n
Cnw479 nw479 0 2f
CT1252 t1252 0 0.1f
M3461 t1252 nw292 vdd vdd pch w=2u l=180n
M3462 t1252 nw186 vdd vdd pch w=2u l=180n
CT1253 t1253 0 0.1f
M3463 t1252 nw292 t1253 0 nch w=1u l=180n
M3464 t1253 nw186 0 0 nch w=1u l=180n
M3465 nw480 t1252 vdd vdd pch w=2u l=180n
M3466 nw480 t1252 0 0 nch w=1u l=180n
Cnw480 nw480 0 2f
CT1254 t1254 0 0.1f
M3467 t1254 nw293 0 0 nch w=1u l=180n
M3468 t1254 nw187 0 0 nch w=1u l=180n
CT1255 t1255 0 0.1f
M3469 t1255 nw293 vdd vdd pch w=2u l=180n
M3470 t1254 nw187 t1255 vdd pch w=2u l=180n
M3471 nw481 t1254 vdd vdd pch w=2u l=180n
M3472 nw481 t1254 0 0 nch w=1u l=180n
Cnw481 nw481 0 2f
CT1256 t1256 0 0.1f
CT1257 t1257 0 0.1f
CT1258 t1258 0 0.1f
M3473 t1256 nw294 vdd vdd pch w=2u l=180n
M3474 t1256 nw188 vdd vdd pch w=2u l=180n
CT1259 t1259 0 0.1f
M3475 t1256 nw294 t1259 0 nch w=1u l=180n
M3476 t1259 nw188 0 0 nch w=1u l=180n
M3477 t1257 nw294 vdd vdd pch w=2u l=180n
M3478 t1257 t1256 vdd vdd pch w=2u l=180n
CT1260 t1260 0 0.1f
M3479 t1257 nw294 t1260 0 nch w=1u l=180n
M3480 t1260 t1256 0 0 nch w=1u l=180n
M3481 t1258 nw188 vdd vdd pch w=2u l=180n
M3482 t1258 t1256 vdd vdd pch w=2u l=180n
CT1261 t1261 0 0.1f
M3483 t1258 nw188 t1261 0 nch w=1u l=180n
M3484 t1261 t1256 0 0 nch w=1u l=180n
M3485 nw482 t1257 vdd vdd pch w=2u l=180n
M3486 nw482 t1258 vdd vdd pch w=2u l=180n
CT1262 t1262 0 0.1f
M3487 nw482 t1257 t1262 0 nch w=1u l=180n
M3488 t1262 t1258 0 0 nch w=1u l=180n
Cnw482 nw482 0 2f
M3489 nw483 nw295 vdd vdd pch w=2u l=180n
M3490 nw483 nw189 vdd vdd pch w=2u l=180n
CT1263 t1263 0 0.1f
M3491 nw483 nw295 t1263 0 nch w=1u l=180n
M3492 t1263 nw189 0 0 nch w=1u l=180n
Cnw483 nw483 0 2f
M3493 nw484 nw296 0 0 nch w=1u l=180n
M3494 nw484 nw190 0 0 nch w=1u l=180n
CT1264 t1264 0 0.1f
M3495 t1264 nw296 vdd vdd pch w=2u l=180n
M3496 nw484 nw190 t1264 vdd pch w=2u l=180n
Cnw484 nw484 0 2f
CT1265 t1265 0 0.1f
M3497 t1265 nw297 vdd vdd pch w=2u l=180n
M3498 t1265 nw191 vdd vdd pch w=2u l=180n
CT1266 t1266 0 0.1f
M3499 t1265 nw297 t1266 0 nch w=1u l=180n
M3500 t1266 nw191 0 0 nch w=1u l=180n
M3501 nw485 t1265 vdd vdd pch w=2u l=180n
M3502 nw485 t1265 0 0 nch w=1u l=180n
Cnw485 nw485 0 2f
CT1267 t1267 0 0.1f
M3503 t1267 nw298 0 0 nch w=1u l=180n
M3504 t1267 nw192 0 0 nch w=1u l=180n
CT1268 t1268 0 0.1f
M3505 t1268 nw298 vdd vdd pch w=2u l=180n
M3506 t1267 nw192 t1268 vdd pch w=2u l=180n
M3507 nw486 t1267 vdd vdd pch w=2u l=180n
M3508 nw486 t1267 0 0 nch w=1u l=180n
Cnw486 nw486 0 2f
CT1269 t1269 0 0.1f
CT1270 t1270 0 0.1f
CT1271 t1271 0 0.1f
M3509 t1269 nw299 vdd vdd pch w=2u l=180n
M3510 t1269 nw193 vdd vdd pch w=2u l=180n
CT1272 t1272 0 0.1f
M3511 t1269 nw299 t1272 0 nch w=1u l=180n
M3512 t1272 nw193 0 0 nch w=1u l=180n
M3513 t1270 nw299 vdd vdd pch w=2u l=180n
M3514 t1270 t1269 vdd vdd pch w=2u l=180n
CT1273 t1273 0 0.1f
M3515 t1270 nw299 t1273 0 nch w=1u l=180n
M3516 t1273 t1269 0 0 nch w=1u l=180n
M3517 t1271 nw193 vdd vdd pch w=2u l=180n
M3518 t1271 t1269 vdd vdd pch w=2u l=180n
CT1274 t1274 0 0.1f
M3519 t1271 nw193 t1274 0 nch w=1u l=180n
M3520 t1274 t1269 0 0 nch w=1u l=180n
M3521 nw487 t1270 vdd vdd pch w=2u l=180n
M3522 nw487 t1271 vdd vdd pch w=2u l=180n
CT1275 t1275 0 0.1f
M3523 nw487 t1270 t1275 0 nch w=1u l=180n
M3524 t1275 t1271 0 0 nch w=1u l=180n
Cnw487 nw487 0 2f
M3525 nw488 nw300 vdd vdd pch w=2u l=180n
M3526 nw488 nw194 vdd vdd pch w=2u l=180n
CT1276 t1276 0 0.1f
M3527 nw488 nw300 t1276 0 nch w=1u l=180n
M3528 t1276 nw194 0 0 nch w=1u l=180n
Cnw488 nw488 0 2f
M3529 nw489 nw301 0 0 nch w=1u l=180n
M3530 nw489 nw195 0 0 nch w=1u l=180n
CT1277 t1277 0 0.1f
M3531 t1277 nw301 vdd vdd pch w=2u l=180n
M3532 nw489 nw195 t1277 vdd pch w=2u l=180n
Cnw489 nw489 0 2f
CT1278 t1278 0 0.1f
M3533 t1278 nw302 vdd vdd pch w=2u l=180n
M3534 t1278 nw196 vdd vdd pch w=2u l=180n
CT1279 t1279 0 0.1f
M3535 t1278 nw302 t1279 0 nch w=1u l=180n
M3536 t1279 nw196 0 0 nch w=1u l=180n
M3537 nw490 t1278 vdd vdd pch w=2u l=180n
M3538 nw490 t1278 0 0 nch w=1u l=180n
Cnw490 nw490 0 2f
CT1280 t1280 0 0.1f
M3539 t1280 nw303 0 0 nch w=1u l=180n
M3540 t1280 nw197 0 0 nch w=1u l=180n
CT1281 t1281 0 0.1f
M3541 t1281 nw303 vdd vdd pch w=2u l=180n
M3542 t1280 nw197 t1281 vdd pch w=2u l=180n
M3543 nw491 t1280 vdd vdd pch w=2u l=180n
M3544 nw491 t1280 0 0 nch w=1u l=180n
Cnw491 nw491 0 2f
CT1282 t1282 0 0.1f
CT1283 t1283 0 0.1f
CT1284 t1284 0 0.1f
M3545 t1282 nw304 vdd vdd pch w=2u l=180n
M3546 t1282 nw198 vdd vdd pch w=2u l=180n
CT1285 t1285 0 0.1f
M3547 t1282 nw304 t1285 0 nch w=1u l=180n
M3548 t1285 nw198 0 0 nch w=1u l=180n
M3549 t1283 nw304 vdd vdd pch w=2u l=180n
M3550 t1283 t1282 vdd vdd pch w=2u l=180n
CT1286 t1286 0 0.1f
M3551 t1283 nw304 t1286 0 nch w=1u l=180n
M3552 t1286 t1282 0 0 nch w=1u l=180n
M3553 t1284 nw198 vdd vdd pch w=2u l=180n
M3554 t1284 t1282 vdd vdd pch w=2u l=180n
CT1287 t1287 0 0.1f
M3555 t1284 nw198 t1287 0 nch w=1u l=180n
M3556 t1287 t1282 0 0 nch w=1u l=180n
M3557 nw492 t1283 vdd vdd pch w=2u l=180n
M3558 nw492 t1284 vdd vdd pch w=2u l=180n
CT1288 t1288 0 0.1f
M3559 nw492 t1283 t1288 0 nch w=1u l=180n
M3560 t1288 t1284 0 0 nch w=1u l=180n
Cnw492 nw492 0 2f
M3561 nw493 nw305 vdd vdd pch w=2u l=180n
M3562 nw493 nw199 vdd vdd pch w=2u l=180n
CT1289 t1289 0 0.1f
M3563 nw493 nw305 t1289 0 nch w=1u l=180n
M3564 t1289 nw199 0 0 nch w=1u l=180n
Cnw493 nw493 0 2f
M3565 nw494 nw306 0 0 nch w=1u l=180n
M3566 nw494 nw200 0 0 nch w=1u l=180n
CT1290 t1290 0 0.1f
M3567 t1290 nw306 vdd vdd pch w=2u l=180n
M3568 nw494 nw200 t1290 vdd pch w=2u l=180n
Cnw494 nw494 0 2f
CT1291 t1291 0 0.1f
M3569 t1291 nw307 vdd vdd pch w=2u l=180n
M3570 t1291 nw201 vdd vdd pch w=2u l=180n
CT1292 t1292 0 0.1f
M3571 t1291 nw307 t1292 0 nch w=1u l=180n
M3572 t1292 nw201 0 0 nch w=1u l=180n
M3573 nw495 t1291 vdd vdd pch w=2u l=180n
M3574 nw495 t1291 0 0 nch w=1u l=180n
Cnw495 nw495 0 2f
CT1293 t1293 0 0.1f
M3575 t1293 nw308 0 0 nch w=1u l=180n
M3576 t1293 nw202 0 0 nch w=1u l=180n
CT1294 t1294 0 0.1f
M3577 t1294 nw308 vdd vdd pch w=2u l=180n
M3578 t1293 nw202 t1294 vdd pch w=2u l=180n
M3579 nw496 t1293 vdd vdd pch w=2u l=180n
M3580 nw496 t1293 0 0 nch w=1u l=180n
Cnw496 nw496 0 2f
CT1295 t1295 0 0.1f
CT1296 t1296 0 0.1f
CT1297 t1297 0 0.1f
M3581 t1295 nw309 vdd vdd pch w=2u l=180n
M3582 t1295 nw203 vdd vdd pch w=2u l=180n
CT1298 t1298 0 0.1f
M3583 t1295 nw309 t1298 0 nch w=1u l=180n
M3584 t1298 nw203 0 0 nch w=1u l=180n
M3585 t1296 nw309 vdd vdd pch w=2u l=180n
M3586 t1296 t1295 vdd vdd pch w=2u l=180n
CT1299 t1299 0 0.1f
M3587 t1296 nw309 t1299 0 nch w=1u l=180n
M3588 t1299 t1295 0 0 nch w=1u l=180n
M3589 t1297 nw203 vdd vdd pch w=2u l=180n
M3590 t1297 t1295 vdd vdd pch w=2u l=180n
CT1300 t1300 0 0.1f
M3591 t1297 nw203 t1300 0 nch w=1u l=180n
M3592 t1300 t1295 0 0 nch w=1u l=180n
M3593 nw497 t1296 vdd vdd pch w=2u l=180n
M3594 nw497 t1297 vdd vdd pch w=2u l=180n
CT1301 t1301 0 0.1f
M3595 nw497 t1296 t1301 0 nch w=1u l=180n
M3596 t1301 t1297 0 0 nch w=1u l=180n
Cnw497 nw497 0 2f
M3597 nw498 nw310 vdd vdd pch w=2u l=180n
M3598 nw498 nw204 vdd vdd pch w=2u l=180n
CT1302 t1302 0 0.1f
M3599 nw498 nw310 t1302 0 nch w=1u l=180n
M3600 t1302 nw204 0 0 nch w=1u l=180n
Cnw498 nw498 0 2f
M3601 nw499 nw311 0 0 nch w=1u l=180n
M3602 nw499 nw205 0 0 nch w=1u l=180n
CT1303 t1303 0 0.1f
M3603 t1303 nw311 vdd vdd pch w=2u l=180n
M3604 nw499 nw205 t1303 vdd pch w=2u l=180n
Cnw499 nw499 0 2f
CT1304 t1304 0 0.1f
M3605 t1304 nw312 vdd vdd pch w=2u l=180n
M3606 t1304 nw206 vdd vdd pch w=2u l=180n
CT1305 t1305 0 0.1f
M3607 t1304 nw312 t1305 0 nch w=1u l=180n
M3608 t1305 nw206 0 0 nch w=1u l=180n
M3609 nw500 t1304 vdd vdd pch w=2u l=180n
M3610 nw500 t1304 0 0 nch w=1u l=180n
Cnw500 nw500 0 2f
CT1306 t1306 0 0.1f
M3611 t1306 nw313 0 0 nch w=1u l=180n
M3612 t1306 nw207 0 0 nch w=1u l=180n
CT1307 t1307 0 0.1f
M3613 t1307 nw313 vdd vdd pch w=2u l=180n
M3614 t1306 nw207 t1307 vdd pch w=2u l=180n
M3615 nw501 t1306 vdd vdd pch w=2u l=180n
M3616 nw501 t1306 0 0 nch w=1u l=180n
Cnw501 nw501 0 2f
CT1308 t1308 0 0.1f
CT1309 t1309 0 0.1f
CT1310 t1310 0 0.1f
M3617 t1308 nw314 vdd vdd pch w=2u l=180n
M3618 t1308 nw208 vdd vdd pch w=2u l=180n
CT1311 t1311 0 0.1f
M3619 t1308 nw314 t1311 0 nch w=1u l=180n
M3620 t1311 nw208 0 0 nch w=1u l=180n
M3621 t1309 nw314 vdd vdd pch w=2u l=180n
M3622 t1309 t1308 vdd vdd pch w=2u l=180n
CT1312 t1312 0 0.1f
M3623 t1309 nw314 t1312 0 nch w=1u l=180n
M3624 t1312 t1308 0 0 nch w=1u l=180n
M3625 t1310 nw208 vdd vdd pch w=2u l=180n
M3626 t1310 t1308 vdd vdd pch w=2u l=180n
CT1313 t1313 0 0.1f
M3627 t1310 nw208 t1313 0 nch w=1u l=180n
M3628 t1313 t1308 0 0 nch w=1u l=180n
M3629 nw502 t1309 vdd vdd pch w=2u l=180n
M3630 nw502 t1310 vdd vdd pch w=2u l=180n
CT1314 t1314 0 0.1f
M3631 nw502 t1309 t1314 0 nch w=1u l=180n
M3632 t1314 t1310 0 0 nch w=1u l=180n
Cnw502 nw502 0 2f
CT1315 t1315 0 0.1f
M3633 t1315 nw502 vdd vdd pch w=2u l=180n
M3634 t1315 nw502 0 0 nch w=1u l=180n
M3635 no0 t1315 vdd vdd pch w=2u l=180n
M3636 no0 t1315 0 0 nch w=1u l=180n
Cno0 no0 0 2f
CT1316 t1316 0 0.1f
M3637 t1316 nw501 vdd vdd pch w=2u l=180n
M3638 t1316 nw501 0 0 nch w=1u l=180n
M3639 no1 t1316 vdd vdd pch w=2u l=180n
M3640 no1 t1316 0 0 nch w=1u l=180n
Cno1 no1 0 2f
CT1317 t1317 0 0.1f
M3641 t1317 nw500 vdd vdd pch w=2u l=180n
M3642 t1317 nw500 0 0 nch w=1u l=180n
M3643 no2 t1317 vdd vdd pch w=2u l=180n
M3644 no2 t1317 0 0 nch w=1u l=180n
Cno2 no2 0 2f
CT1318 t1318 0 0.1f
M3645 t1318 nw499 vdd vdd pch w=2u l=180n
M3646 t1318 nw499 0 0 nch w=1u l=180n
M3647 no3 t1318 vdd vdd pch w=2u l=180n
M3648 no3 t1318 0 0 nch w=1u l=180n
Cno3 no3 0 2f
CT1319 t1319 0 0.1f
M3649 t1319 nw498 vdd vdd pch w=2u l=180n
M3650 t1319 nw498 0 0 nch w=1u l=180n
M3651 no4 t1319 vdd vdd pch w=2u l=180n
M3652 no4 t1319 0 0 nch w=1u l=180n
Cno4 no4 0 2f
CT1320 t1320 0 0.1f
M3653 t1320 nw497 vdd vdd pch w=2u l=180n
M3654 t1320 nw497 0 0 nch w=1u l=180n
M3655 no5 t1320 vdd vdd pch w=2u l=180n
M3656 no5 t1320 0 0 nch w=1u l=180n
Cno5 no5 0 2f
CT1321 t1321 0 0.1f
M3657 t1321 nw496 vdd vdd pch w=2u l=180n
M3658 t1321 nw496 0 0 nch w=1u l=180n
M3659 no6 t1321 vdd vdd pch w=2u l=180n
M3660 no6 t1321 0 0 nch w=1u l=180n
Cno6 no6 0 2f
CT1322 t1322 0 0.1f
M3661 t1322 nw495 vdd vdd pch w=2u l=180n
M3662 t1322 nw495 0 0 nch w=1u l=180n
M3663 no7 t1322 vdd vdd pch w=2u l=180n
M3664 no7 t1322 0 0 nch w=1u l=180n
Cno7 no7 0 2f
.model nch NMOS (vto=0.45 kp=200u lambda=0.05)
.model pch PMOS (vto=-0.45 kp=100u lambda=0.05)
* outputs: nw2 nq0 nq1 nq2 nq3 nq4 nq5 nq6 nq7 nq8 nq9 nq10 nq11 nq12 nq13 nq14 nq15 nq16 no0 no1 no2 no3 no4 no5 no6 no7
.end
