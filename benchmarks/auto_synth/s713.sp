* s713 (s713: 19 flip-flops, 393 gates): 464 gates, 3148 transistors
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
VIN27 nq18 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
M1 nw1 ni0 vdd vdd pch w=2u l=180n
M2 nw1 ni0 0 0 nch w=1u l=180n
Cnw1 nw1 0 2f
CT1 t1 0 0.1f
M3 t1 ni1 vdd vdd pch w=2u l=180n
M4 t1 nw1 vdd vdd pch w=2u l=180n
CT2 t2 0 0.1f
M5 t1 ni1 t2 0 nch w=1u l=180n
M6 t2 nw1 0 0 nch w=1u l=180n
M7 nw2 t1 vdd vdd pch w=2u l=180n
M8 nw2 t1 0 0 nch w=1u l=180n
Cnw2 nw2 0 2f
CT3 t3 0 0.1f
M9 t3 ni0 vdd vdd pch w=2u l=180n
M10 t3 ni0 vdd vdd pch w=2u l=180n
CT4 t4 0 0.1f
M11 t3 ni0 t4 0 nch w=1u l=180n
M12 t4 ni0 0 0 nch w=1u l=180n
M13 nw3 t3 vdd vdd pch w=2u l=180n
M14 nw3 t3 0 0 nch w=1u l=180n
Cnw3 nw3 0 2f
CT5 t5 0 0.1f
M15 t5 nw2 0 0 nch w=1u l=180n
M16 t5 nw3 0 0 nch w=1u l=180n
CT6 t6 0 0.1f
M17 t6 nw2 vdd vdd pch w=2u l=180n
M18 t5 nw3 t6 vdd pch w=2u l=180n
M19 nw4 t5 vdd vdd pch w=2u l=180n
M20 nw4 t5 0 0 nch w=1u l=180n
Cnw4 nw4 0 2f
M21 nw5 ni0 vdd vdd pch w=2u l=180n
M22 nw5 ni0 0 0 nch w=1u l=180n
Cnw5 nw5 0 2f
CT7 t7 0 0.1f
M23 t7 nq0 vdd vdd pch w=2u l=180n
M24 t7 nw5 vdd vdd pch w=2u l=180n
CT8 t8 0 0.1f
M25 t7 nq0 t8 0 nch w=1u l=180n
M26 t8 nw5 0 0 nch w=1u l=180n
M27 nw6 t7 vdd vdd pch w=2u l=180n
M28 nw6 t7 0 0 nch w=1u l=180n
Cnw6 nw6 0 2f
CT9 t9 0 0.1f
M29 t9 ni1 vdd vdd pch w=2u l=180n
M30 t9 ni0 vdd vdd pch w=2u l=180n
CT10 t10 0 0.1f
M31 t9 ni1 t10 0 nch w=1u l=180n
M32 t10 ni0 0 0 nch w=1u l=180n
M33 nw7 t9 vdd vdd pch w=2u l=180n
M34 nw7 t9 0 0 nch w=1u l=180n
Cnw7 nw7 0 2f
CT11 t11 0 0.1f
M35 t11 nw6 0 0 nch w=1u l=180n
M36 t11 nw7 0 0 nch w=1u l=180n
CT12 t12 0 0.1f
M37 t12 nw6 vdd vdd pch w=2u l=180n
M38 t11 nw7 t12 vdd pch w=2u l=180n
M39 nw8 t11 vdd vdd pch w=2u l=180n
M40 nw8 t11 0 0 nch w=1u l=180n
Cnw8 nw8 0 2f
M41 nw9 ni0 vdd vdd pch w=2u l=180n
M42 nw9 ni0 0 0 nch w=1u l=180n
Cnw9 nw9 0 2f
CT13 t13 0 0.1f
M43 t13 nq1 vdd vdd pch w=2u l=180n
M44 t13 nw9 vdd vdd pch w=2u l=180n
CT14 t14 0 0.1f
M45 t13 nq1 t14 0 nch w=1u l=180n
M46 t14 nw9 0 0 nch w=1u l=180n
M47 nw10 t13 vdd vdd pch w=2u l=180n
M48 nw10 t13 0 0 nch w=1u l=180n
Cnw10 nw10 0 2f
CT15 t15 0 0.1f
M49 t15 ni2 vdd vdd pch w=2u l=180n
M50 t15 ni0 vdd vdd pch w=2u l=180n
CT16 t16 0 0.1f
M51 t15 ni2 t16 0 nch w=1u l=180n
M52 t16 ni0 0 0 nch w=1u l=180n
M53 nw11 t15 vdd vdd pch w=2u l=180n
M54 nw11 t15 0 0 nch w=1u l=180n
Cnw11 nw11 0 2f
CT17 t17 0 0.1f
M55 t17 nw10 0 0 nch w=1u l=180n
M56 t17 nw11 0 0 nch w=1u l=180n
CT18 t18 0 0.1f
M57 t18 nw10 vdd vdd pch w=2u l=180n
M58 t17 nw11 t18 vdd pch w=2u l=180n
M59 nw12 t17 vdd vdd pch w=2u l=180n
M60 nw12 t17 0 0 nch w=1u l=180n
Cnw12 nw12 0 2f
M61 nw13 ni0 vdd vdd pch w=2u l=180n
M62 nw13 ni0 0 0 nch w=1u l=180n
Cnw13 nw13 0 2f
CT19 t19 0 0.1f
M63 t19 nq2 vdd vdd pch w=2u l=180n
M64 t19 nw13 vdd vdd pch w=2u l=180n
CT20 t20 0 0.1f
M65 t19 nq2 t20 0 nch w=1u l=180n
M66 t20 nw13 0 0 nch w=1u l=180n
M67 nw14 t19 vdd vdd pch w=2u l=180n
M68 nw14 t19 0 0 nch w=1u l=180n
Cnw14 nw14 0 2f
CT21 t21 0 0.1f
M69 t21 ni3 vdd vdd pch w=2u l=180n
M70 t21 ni0 vdd vdd pch w=2u l=180n
CT22 t22 0 0.1f
M71 t21 ni3 t22 0 nch w=1u l=180n
M72 t22 ni0 0 0 nch w=1u l=180n
M73 nw15 t21 vdd vdd pch w=2u l=180n
M74 nw15 t21 0 0 nch w=1u l=180n
Cnw15 nw15 0 2f
CT23 t23 0 0.1f
M75 t23 nw14 0 0 nch w=1u l=180n
M76 t23 nw15 0 0 nch w=1u l=180n
CT24 t24 0 0.1f
M77 t24 nw14 vdd vdd pch w=2u l=180n
M78 t23 nw15 t24 vdd pch w=2u l=180n
M79 nw16 t23 vdd vdd pch w=2u l=180n
M80 nw16 t23 0 0 nch w=1u l=180n
Cnw16 nw16 0 2f
M81 nw17 ni0 vdd vdd pch w=2u l=180n
M82 nw17 ni0 0 0 nch w=1u l=180n
Cnw17 nw17 0 2f
CT25 t25 0 0.1f
M83 t25 nq3 vdd vdd pch w=2u l=180n
M84 t25 nw17 vdd vdd pch w=2u l=180n
CT26 t26 0 0.1f
M85 t25 nq3 t26 0 nch w=1u l=180n
M86 t26 nw17 0 0 nch w=1u l=180n
M87 nw18 t25 vdd vdd pch w=2u l=180n
M88 nw18 t25 0 0 nch w=1u l=180n
Cnw18 nw18 0 2f
CT27 t27 0 0.1f
M89 t27 ni4 vdd vdd pch w=2u l=180n
M90 t27 ni0 vdd vdd pch w=2u l=180n
CT28 t28 0 0.1f
M91 t27 ni4 t28 0 nch w=1u l=180n
M92 t28 ni0 0 0 nch w=1u l=180n
M93 nw19 t27 vdd vdd pch w=2u l=180n
M94 nw19 t27 0 0 nch w=1u l=180n
Cnw19 nw19 0 2f
CT29 t29 0 0.1f
M95 t29 nw18 0 0 nch w=1u l=180n
M96 t29 nw19 0 0 nch w=1u l=180n
CT30 t30 0 0.1f
M97 t30 nw18 vdd vdd pch w=2u l=180n
M98 t29 nw19 t30 vdd pch w=2u l=180n
M99 nw20 t29 vdd vdd pch w=2u l=180n
M100 nw20 t29 0 0 nch w=1u l=180n
Cnw20 nw20 0 2f
M101 nw21 ni0 vdd vdd pch w=2u l=180n
M102 nw21 ni0 0 0 nch w=1u l=180n
Cnw21 nw21 0 2f
CT31 t31 0 0.1f
M103 t31 nq4 vdd vdd pch w=2u l=180n
M104 t31 nw21 vdd vdd pch w=2u l=180n
CT32 t32 0 0.1f
M105 t31 nq4 t32 0 nch w=1u l=180n
M106 t32 nw21 0 0 nch w=1u l=180n
M107 nw22 t31 vdd vdd pch w=2u l=180n
M108 nw22 t31 0 0 nch w=1u l=180n
Cnw22 nw22 0 2f
CT33 t33 0 0.1f
M109 t33 ni5 vdd vdd pch w=2u l=180n
M110 t33 ni0 vdd vdd pch w=2u l=180n
CT34 t34 0 0.1f
M111 t33 ni5 t34 0 nch w=1u l=180n
M112 t34 ni0 0 0 nch w=1u l=180n
M113 nw23 t33 vdd vdd pch w=2u l=180n
M114 nw23 t33 0 0 nch w=1u l=180n
Cnw23 nw23 0 2f
CT35 t35 0 0.1f
M115 t35 nw22 0 0 nch w=1u l=180n
M116 t35 nw23 0 0 nch w=1u l=180n
CT36 t36 0 0.1f
M117 t36 nw22 vdd vdd pch w=2u l=180n
M118 t35 nw23 t36 vdd pch w=2u l=180n
M119 nw24 t35 vdd vdd pch w=2u l=180n
M120 nw24 t35 0 0 nch w=1u l=180n
Cnw24 nw24 0 2f
M121 nw25 ni0 vdd vdd pch w=2u l=180n
M122 nw25 ni0 0 0 nch w=1u l=180n
Cnw25 nw25 0 2f
CT37 t37 0 0.1f
M123 t37 nq5 vdd vdd pch w=2u l=180n
M124 t37 nw25 vdd vdd pch w=2u l=180n
CT38 t38 0 0.1f
M125 t37 nq5 t38 0 nch w=1u l=180n
M126 t38 nw25 0 0 nch w=1u l=180n
M127 nw26 t37 vdd vdd pch w=2u l=180n
M128 nw26 t37 0 0 nch w=1u l=180n
Cnw26 nw26 0 2f
CT39 t39 0 0.1f
M129 t39 ni6 vdd vdd pch w=2u l=180n
M130 t39 ni0 vdd vdd pch w=2u l=180n
CT40 t40 0 0.1f
M131 t39 ni6 t40 0 nch w=1u l=180n
M132 t40 ni0 0 0 nch w=1u l=180n
M133 nw27 t39 vdd vdd pch w=2u l=180n
M134 nw27 t39 0 0 nch w=1u l=180n
Cnw27 nw27 0 2f
CT41 t41 0 0.1f
M135 t41 nw26 0 0 nch w=1u l=180n
M136 t41 nw27 0 0 nch w=1u l=180n
CT42 t42 0 0.1f
M137 t42 nw26 vdd vdd pch w=2u l=180n
M138 t41 nw27 t42 vdd pch w=2u l=180n
M139 nw28 t41 vdd vdd pch w=2u l=180n
M140 nw28 t41 0 0 nch w=1u l=180n
Cnw28 nw28 0 2f
M141 nw29 ni0 vdd vdd pch w=2u l=180n
M142 nw29 ni0 0 0 nch w=1u l=180n
Cnw29 nw29 0 2f
CT43 t43 0 0.1f
M143 t43 nq6 vdd vdd pch w=2u l=180n
M144 t43 nw29 vdd vdd pch w=2u l=180n
CT44 t44 0 0.1f
M145 t43 nq6 t44 0 nch w=1u l=180n
M146 t44 nw29 0 0 nch w=1u l=180n
M147 nw30 t43 vdd vdd pch w=2u l=180n
M148 nw30 t43 0 0 nch w=1u l=180n
Cnw30 nw30 0 2f
CT45 t45 0 0.1f
M149 t45 ni7 vdd vdd pch w=2u l=180n
M150 t45 ni0 vdd vdd pch w=2u l=180n
CT46 t46 0 0.1f
M151 t45 ni7 t46 0 nch w=1u l=180n
M152 t46 ni0 0 0 nch w=1u l=180n
M153 nw31 t45 vdd vdd pch w=2u l=180n
M154 nw31 t45 0 0 nch w=1u l=180n
Cnw31 nw31 0 2f
CT47 t47 0 0.1f
M155 t47 nw30 0 0 nch w=1u l=180n
M156 t47 nw31 0 0 nch w=1u l=180n
CT48 t48 0 0.1f
M157 t48 nw30 vdd vdd pch w=2u l=180n
M158 t47 nw31 t48 vdd pch w=2u l=180n
M159 nw32 t47 vdd vdd pch w=2u l=180n
M160 nw32 t47 0 0 nch w=1u l=180n
Cnw32 nw32 0 2f
M161 nw33 ni0 vdd vdd pch w=2u l=180n
M162 nw33 ni0 0 0 nch w=1u l=180n
Cnw33 nw33 0 2f
CT49 t49 0 0.1f
M163 t49 nq7 vdd vdd pch w=2u l=180n
M164 t49 nw33 vdd vdd pch w=2u l=180n
CT50 t50 0 0.1f
M165 t49 nq7 t50 0 nch w=1u l=180n
M166 t50 nw33 0 0 nch w=1u l=180n
M167 nw34 t49 vdd vdd pch w=2u l=180n
M168 nw34 t49 0 0 nch w=1u l=180n
Cnw34 nw34 0 2f
CT51 t51 0 0.1f
M169 t51 ni8 vdd vdd pch w=2u l=180n
M170 t51 ni0 vdd vdd pch w=2u l=180n
CT52 t52 0 0.1f
M171 t51 ni8 t52 0 nch w=1u l=180n
M172 t52 ni0 0 0 nch w=1u l=180n
M173 nw35 t51 vdd vdd pch w=2u l=180n
M174 nw35 t51 0 0 nch w=1u l=180n
Cnw35 nw35 0 2f
CT53 t53 0 0.1f
M175 t53 nw34 0 0 nch w=1u l=180n
M176 t53 nw35 0 0 nch w=1u l=180n
CT54 t54 0 0.1f
M177 t54 nw34 vdd vdd pch w=2u l=180n
M178 t53 nw35 t54 vdd pch w=2u l=180n
M179 nw36 t53 vdd vdd pch w=2u l=180n
M180 nw36 t53 0 0 nch w=1u l=180n
Cnw36 nw36 0 2f
M181 nw37 ni0 vdd vdd pch w=2u l=180n
M182 nw37 ni0 0 0 nch w=1u l=180n
Cnw37 nw37 0 2f
CT55 t55 0 0.1f
M183 t55 nq8 vdd vdd pch w=2u l=180n
M184 t55 nw37 vdd vdd pch w=2u l=180n
CT56 t56 0 0.1f
M185 t55 nq8 t56 0 nch w=1u l=180n
M186 t56 nw37 0 0 nch w=1u l=180n
M187 nw38 t55 vdd vdd pch w=2u l=180n
M188 nw38 t55 0 0 nch w=1u l=180n
Cnw38 nw38 0 2f
CT57 t57 0 0.1f
M189 t57 ni0 vdd vdd pch w=2u l=180n
M190 t57 ni0 vdd vdd pch w=2u l=180n
CT58 t58 0 0.1f
M191 t57 ni0 t58 0 nch w=1u l=180n
M192 t58 ni0 0 0 nch w=1u l=180n
M193 nw39 t57 vdd vdd pch w=2u l=180n
M194 nw39 t57 0 0 nch w=1u l=180n
Cnw39 nw39 0 2f
CT59 t59 0 0.1f
M195 t59 nw38 0 0 nch w=1u l=180n
M196 t59 nw39 0 0 nch w=1u l=180n
CT60 t60 0 0.1f
M197 t60 nw38 vdd vdd pch w=2u l=180n
M198 t59 nw39 t60 vdd pch w=2u l=180n
M199 nw40 t59 vdd vdd pch w=2u l=180n
M200 nw40 t59 0 0 nch w=1u l=180n
Cnw40 nw40 0 2f
M201 nw41 ni0 vdd vdd pch w=2u l=180n
M202 nw41 ni0 0 0 nch w=1u l=180n
Cnw41 nw41 0 2f
CT61 t61 0 0.1f
M203 t61 nq9 vdd vdd pch w=2u l=180n
M204 t61 nw41 vdd vdd pch w=2u l=180n
CT62 t62 0 0.1f
M205 t61 nq9 t62 0 nch w=1u l=180n
M206 t62 nw41 0 0 nch w=1u l=180n
M207 nw42 t61 vdd vdd pch w=2u l=180n
M208 nw42 t61 0 0 nch w=1u l=180n
Cnw42 nw42 0 2f
CT63 t63 0 0.1f
M209 t63 ni1 vdd vdd pch w=2u l=180n
M210 t63 ni0 vdd vdd pch w=2u l=180n
CT64 t64 0 0.1f
M211 t63 ni1 t64 0 nch w=1u l=180n
M212 t64 ni0 0 0 nch w=1u l=180n
M213 nw43 t63 vdd vdd pch w=2u l=180n
M214 nw43 t63 0 0 nch w=1u l=180n
Cnw43 nw43 0 2f
CT65 t65 0 0.1f
M215 t65 nw42 0 0 nch w=1u l=180n
M216 t65 nw43 0 0 nch w=1u l=180n
CT66 t66 0 0.1f
M217 t66 nw42 vdd vdd pch w=2u l=180n
M218 t65 nw43 t66 vdd pch w=2u l=180n
M219 nw44 t65 vdd vdd pch w=2u l=180n
M220 nw44 t65 0 0 nch w=1u l=180n
Cnw44 nw44 0 2f
M221 nw45 ni0 vdd vdd pch w=2u l=180n
M222 nw45 ni0 0 0 nch w=1u l=180n
Cnw45 nw45 0 2f
CT67 t67 0 0.1f
M223 t67 nq10 vdd vdd pch w=2u l=180n
M224 t67 nw45 vdd vdd pch w=2u l=180n
CT68 t68 0 0.1f
M225 t67 nq10 t68 0 nch w=1u l=180n
M226 t68 nw45 0 0 nch w=1u l=180n
M227 nw46 t67 vdd vdd pch w=2u l=180n
M228 nw46 t67 0 0 nch w=1u l=180n
Cnw46 nw46 0 2f
CT69 t69 0 0.1f
M229 t69 ni2 vdd vdd pch w=2u l=180n
M230 t69 ni0 vdd vdd pch w=2u l=180n
CT70 t70 0 0.1f
M231 t69 ni2 t70 0 nch w=1u l=180n
M232 t70 ni0 0 0 nch w=1u l=180n
M233 nw47 t69 vdd vdd pch w=2u l=180n
M234 nw47 t69 0 0 nch w=1u l=180n
Cnw47 nw47 0 2f
CT71 t71 0 0.1f
M235 t71 nw46 0 0 nch w=1u l=180n
M236 t71 nw47 0 0 nch w=1u l=180n
CT72 t72 0 0.1f
M237 t72 nw46 vdd vdd pch w=2u l=180n
M238 t71 nw47 t72 vdd pch w=2u l=180n
M239 nw48 t71 vdd vdd pch w=2u l=180n
M240 nw48 t71 0 0 nch w=1u l=180n
Cnw48 nw48 0 2f
M241 nw49 ni0 vdd vdd pch w=2u l=180n
M242 nw49 ni0 0 0 nch w=1u l=180n
Cnw49 nw49 0 2f
CT73 t73 0 0.1f
M243 t73 nq11 vdd vdd pch w=2u l=180n
M244 t73 nw49 vdd vdd pch w=2u l=180n
CT74 t74 0 0.1f
M245 t73 nq11 t74 0 nch w=1u l=180n
M246 t74 nw49 0 0 nch w=1u l=180n
M247 nw50 t73 vdd vdd pch w=2u l=180n
M248 nw50 t73 0 0 nch w=1u l=180n
Cnw50 nw50 0 2f
CT75 t75 0 0.1f
M249 t75 ni3 vdd vdd pch w=2u l=180n
M250 t75 ni0 vdd vdd pch w=2u l=180n
CT76 t76 0 0.1f
M251 t75 ni3 t76 0 nch w=1u l=180n
M252 t76 ni0 0 0 nch w=1u l=180n
M253 nw51 t75 vdd vdd pch w=2u l=180n
M254 nw51 t75 0 0 nch w=1u l=180n
Cnw51 nw51 0 2f
CT77 t77 0 0.1f
M255 t77 nw50 0 0 nch w=1u l=180n
M256 t77 nw51 0 0 nch w=1u l=180n
CT78 t78 0 0.1f
M257 t78 nw50 vdd vdd pch w=2u l=180n
M258 t77 nw51 t78 vdd pch w=2u l=180n
M259 nw52 t77 vdd vdd pch w=2u l=180n
M260 nw52 t77 0 0 nch w=1u l=180n
Cnw52 nw52 0 2f
M261 nw53 ni0 vdd vdd pch w=2u l=180n
M262 nw53 ni0 0 0 nch w=1u l=180n
Cnw53 nw53 0 2f
CT79 t79 0 0.1f
M263 t79 nq12 vdd vdd pch w=2u l=180n
M264 t79 nw53 vdd vdd pch w=2u l=180n
CT80 t80 0 0.1f
M265 t79 nq12 t80 0 nch w=1u l=180n
M266 t80 nw53 0 0 nch w=1u l=180n
M267 nw54 t79 vdd vdd pch w=2u l=180n
M268 nw54 t79 0 0 nch w=1u l=180n
Cnw54 nw54 0 2f
CT81 t81 0 0.1f
M269 t81 ni4 vdd vdd pch w=2u l=180n
M270 t81 ni0 vdd vdd pch w=2u l=180n
CT82 t82 0 0.1f
M271 t81 ni4 t82 0 nch w=1u l=180n
M272 t82 ni0 0 0 nch w=1u l=180n
M273 nw55 t81 vdd vdd pch w=2u l=180n
M274 nw55 t81 0 0 nch w=1u l=180n
Cnw55 nw55 0 2f
CT83 t83 0 0.1f
M275 t83 nw54 0 0 nch w=1u l=180n
M276 t83 nw55 0 0 nch w=1u l=180n
CT84 t84 0 0.1f
M277 t84 nw54 vdd vdd pch w=2u l=180n
M278 t83 nw55 t84 vdd pch w=2u l=180n
M279 nw56 t83 vdd vdd pch w=2u l=180n
M280 nw56 t83 0 0 nch w=1u l=180n
Cnw56 nw56 0 2f
M281 nw57 ni0 vdd vdd pch w=2u l=180n
M282 nw57 ni0 0 0 nch w=1u l=180n
Cnw57 nw57 0 2f
CT85 t85 0 0.1f
M283 t85 nq13 vdd vdd pch w=2u l=180n
M284 t85 nw57 vdd vdd pch w=2u l=180n
CT86 t86 0 0.1f
M285 t85 nq13 t86 0 nch w=1u l=180n
M286 t86 nw57 0 0 nch w=1u l=180n
M287 nw58 t85 vdd vdd pch w=2u l=180n
M288 nw58 t85 0 0 nch w=1u l=180n
Cnw58 nw58 0 2f
CT87 t87 0 0.1f
M289 t87 ni5 vdd vdd pch w=2u l=180n
M290 t87 ni0 vdd vdd pch w=2u l=180n
CT88 t88 0 0.1f
M291 t87 ni5 t88 0 nch w=1u l=180n
M292 t88 ni0 0 0 nch w=1u l=180n
M293 nw59 t87 vdd vdd pch w=2u l=180n
M294 nw59 t87 0 0 nch w=1u l=180n
Cnw59 nw59 0 2f
CT89 t89 0 0.1f
M295 t89 nw58 0 0 nch w=1u l=180n
M296 t89 nw59 0 0 nch w=1u l=180n
CT90 t90 0 0.1f
M297 t90 nw58 vdd vdd pch w=2u l=180n
M298 t89 nw59 t90 vdd pch w=2u l=180n
M299 nw60 t89 vdd vdd pch w=2u l=180n
M300 nw60 t89 0 0 nch w=1u l=180n
Cnw60 nw60 0 2f
M301 nw61 ni0 vdd vdd pch w=2u l=180n
M302 nw61 ni0 0 0 nch w=1u l=180n
Cnw61 nw61 0 2f
CT91 t91 0 0.1f
M303 t91 nq14 vdd vdd pch w=2u l=180n
M304 t91 nw61 vdd vdd pch w=2u l=180n
CT92 t92 0 0.1f
M305 t91 nq14 t92 0 nch w=1u l=180n
M306 t92 nw61 0 0 nch w=1u l=180n
M307 nw62 t91 vdd vdd pch w=2u l=180n
M308 nw62 t91 0 0 nch w=1u l=180n
Cnw62 nw62 0 2f
CT93 t93 0 0.1f
M309 t93 ni6 vdd vdd pch w=2u l=180n
M310 t93 ni0 vdd vdd pch w=2u l=180n
CT94 t94 0 0.1f
M311 t93 ni6 t94 0 nch w=1u l=180n
M312 t94 ni0 0 0 nch w=1u l=180n
M313 nw63 t93 vdd vdd pch w=2u l=180n
M314 nw63 t93 0 0 nch w=1u l=180n
Cnw63 nw63 0 2f
CT95 t95 0 0.1f
M315 t95 nw62 0 0 nch w=1u l=180n
M316 t95 nw63 0 0 nch w=1u l=180n
CT96 t96 0 0.1f
M317 t96 nw62 vdd vdd pch w=2u l=180n
M318 t95 nw63 t96 vdd pch w=2u l=180n
M319 nw64 t95 vdd vdd pch w=2u l=180n
M320 nw64 t95 0 0 nch w=1u l=180n
Cnw64 nw64 0 2f
M321 nw65 ni0 vdd vdd pch w=2u l=180n
M322 nw65 ni0 0 0 nch w=1u l=180n
Cnw65 nw65 0 2f
CT97 t97 0 0.1f
M323 t97 nq15 vdd vdd pch w=2u l=180n
M324 t97 nw65 vdd vdd pch w=2u l=180n
CT98 t98 0 0.1f
M325 t97 nq15 t98 0 nch w=1u l=180n
M326 t98 nw65 0 0 nch w=1u l=180n
M327 nw66 t97 vdd vdd pch w=2u l=180n
M328 nw66 t97 0 0 nch w=1u l=180n
Cnw66 nw66 0 2f
CT99 t99 0 0.1f
M329 t99 ni7 vdd vdd pch w=2u l=180n
M330 t99 ni0 vdd vdd pch w=2u l=180n
CT100 t100 0 0.1f
M331 t99 ni7 t100 0 nch w=1u l=180n
M332 t100 ni0 0 0 nch w=1u l=180n
M333 nw67 t99 vdd vdd pch w=2u l=180n
M334 nw67 t99 0 0 nch w=1u l=180n
Cnw67 nw67 0 2f
CT101 t101 0 0.1f
M335 t101 nw66 0 0 nch w=1u l=180n
M336 t101 nw67 0 0 nch w=1u l=180n
CT102 t102 0 0.1f
M337 t102 nw66 vdd vdd pch w=2u l=180n
M338 t101 nw67 t102 vdd pch w=2u l=180n
M339 nw68 t101 vdd vdd pch w=2u l=180n
M340 nw68 t101 0 0 nch w=1u l=180n
Cnw68 nw68 0 2f
M341 nw69 ni0 vdd vdd pch w=2u l=180n
M342 nw69 ni0 0 0 nch w=1u l=180n
Cnw69 nw69 0 2f
CT103 t103 0 0.1f
M343 t103 nq16 vdd vdd pch w=2u l=180n
M344 t103 nw69 vdd vdd pch w=2u l=180n
CT104 t104 0 0.1f
M345 t103 nq16 t104 0 nch w=1u l=180n
M346 t104 nw69 0 0 nch w=1u l=180n
M347 nw70 t103 vdd vdd pch w=2u l=180n
M348 nw70 t103 0 0 nch w=1u l=180n
Cnw70 nw70 0 2f
CT105 t105 0 0.1f
M349 t105 ni8 vdd vdd pch w=2u l=180n
M350 t105 ni0 vdd vdd pch w=2u l=180n
CT106 t106 0 0.1f
M351 t105 ni8 t106 0 nch w=1u l=180n
M352 t106 ni0 0 0 nch w=1u l=180n
M353 nw71 t105 vdd vdd pch w=2u l=180n
M354 nw71 t105 0 0 nch w=1u l=180n
Cnw71 nw71 0 2f
CT107 t107 0 0.1f
M355 t107 nw70 0 0 nch w=1u l=180n
M356 t107 nw71 0 0 nch w=1u l=180n
CT108 t108 0 0.1f
M357 t108 nw70 vdd vdd pch w=2u l=180n
M358 t107 nw71 t108 vdd pch w=2u l=180n
M359 nw72 t107 vdd vdd pch w=2u l=180n
M360 nw72 t107 0 0 nch w=1u l=180n
Cnw72 nw72 0 2f
M361 nw73 ni0 vdd vdd pch w=2u l=180n
M362 nw73 ni0 0 0 nch w=1u l=180n
Cnw73 nw73 0 2f
CT109 t109 0 0.1f
M363 t109 nq17 vdd vdd pch w=2u l=180n
M364 t109 nw73 vdd vdd pch w=2u l=180n
CT110 t110 0 0.1f
M365 t109 nq17 t110 0 nch w=1u l=180n
M366 t110 nw73 0 0 nch w=1u l=180n
M367 nw74 t109 vdd vdd pch w=2u l=180n
M368 nw74 t109 0 0 nch w=1u l=180n
Cnw74 nw74 0 2f
CT111 t111 0 0.1f
M369 t111 ni0 vdd vdd pch w=2u l=180n
M370 t111 ni0 vdd vdd pch w=2u l=180n
CT112 t112 0 0.1f
M371 t111 ni0 t112 0 nch w=1u l=180n
M372 t112 ni0 0 0 nch w=1u l=180n
M373 nw75 t111 vdd vdd pch w=2u l=180n
M374 nw75 t111 0 0 nch w=1u l=180n
Cnw75 nw75 0 2f
CT113 t113 0 0.1f
M375 t113 nw74 0 0 nch w=1u l=180n
M376 t113 nw75 0 0 nch w=1u l=180n
CT114 t114 0 0.1f
M377 t114 nw74 vdd vdd pch w=2u l=180n
M378 t113 nw75 t114 vdd pch w=2u l=180n
M379 nw76 t113 vdd vdd pch w=2u l=180n
M380 nw76 t113 0 0 nch w=1u l=180n
Cnw76 nw76 0 2f
M381 nw77 nq1 vdd vdd pch w=2u l=180n
M382 nw77 nq3 vdd vdd pch w=2u l=180n
CT115 t115 0 0.1f
M383 nw77 nq1 t115 0 nch w=1u l=180n
M384 t115 nq3 0 0 nch w=1u l=180n
Cnw77 nw77 0 2f
M385 nw78 nq8 0 0 nch w=1u l=180n
M386 nw78 nq14 0 0 nch w=1u l=180n
CT116 t116 0 0.1f
M387 t116 nq8 vdd vdd pch w=2u l=180n
M388 nw78 nq14 t116 vdd pch w=2u l=180n
Cnw78 nw78 0 2f
CT117 t117 0 0.1f
M389 t117 nq15 vdd vdd pch w=2u l=180n
M390 t117 ni6 vdd vdd pch w=2u l=180n
CT118 t118 0 0.1f
M391 t117 nq15 t118 0 nch w=1u l=180n
M392 t118 ni6 0 0 nch w=1u l=180n
M393 nw79 t117 vdd vdd pch w=2u l=180n
M394 nw79 t117 0 0 nch w=1u l=180n
Cnw79 nw79 0 2f
CT119 t119 0 0.1f
M395 t119 ni3 0 0 nch w=1u l=180n
M396 t119 nq5 0 0 nch w=1u l=180n
CT120 t120 0 0.1f
M397 t120 ni3 vdd vdd pch w=2u l=180n
M398 t119 nq5 t120 vdd pch w=2u l=180n
M399 nw80 t119 vdd vdd pch w=2u l=180n
M400 nw80 t119 0 0 nch w=1u l=180n
Cnw80 nw80 0 2f
CT121 t121 0 0.1f
CT122 t122 0 0.1f
CT123 t123 0 0.1f
M401 t121 nw78 vdd vdd pch w=2u l=180n
M402 t121 nq15 vdd vdd pch w=2u l=180n
CT124 t124 0 0.1f
M403 t121 nw78 t124 0 nch w=1u l=180n
M404 t124 nq15 0 0 nch w=1u l=180n
M405 t122 nw78 vdd vdd pch w=2u l=180n
M406 t122 t121 vdd vdd pch w=2u l=180n
CT125 t125 0 0.1f
M407 t122 nw78 t125 0 nch w=1u l=180n
M408 t125 t121 0 0 nch w=1u l=180n
M409 t123 nq15 vdd vdd pch w=2u l=180n
M410 t123 t121 vdd vdd pch w=2u l=180n
CT126 t126 0 0.1f
M411 t123 nq15 t126 0 nch w=1u l=180n
M412 t126 t121 0 0 nch w=1u l=180n
M413 nw81 t122 vdd vdd pch w=2u l=180n
M414 nw81 t123 vdd vdd pch w=2u l=180n
CT127 t127 0 0.1f
M415 nw81 t122 t127 0 nch w=1u l=180n
M416 t127 t123 0 0 nch w=1u l=180n
Cnw81 nw81 0 2f
M417 nw82 nq3 vdd vdd pch w=2u l=180n
M418 nw82 ni6 vdd vdd pch w=2u l=180n
CT128 t128 0 0.1f
M419 nw82 nq3 t128 0 nch w=1u l=180n
M420 t128 ni6 0 0 nch w=1u l=180n
Cnw82 nw82 0 2f
M421 nw83 nq9 0 0 nch w=1u l=180n
M422 nw83 nq1 0 0 nch w=1u l=180n
CT129 t129 0 0.1f
M423 t129 nq9 vdd vdd pch w=2u l=180n
M424 nw83 nq1 t129 vdd pch w=2u l=180n
Cnw83 nw83 0 2f
CT130 t130 0 0.1f
M425 t130 nq15 vdd vdd pch w=2u l=180n
M426 t130 nq10 vdd vdd pch w=2u l=180n
CT131 t131 0 0.1f
M427 t130 nq15 t131 0 nch w=1u l=180n
M428 t131 nq10 0 0 nch w=1u l=180n
M429 nw84 t130 vdd vdd pch w=2u l=180n
M430 nw84 t130 0 0 nch w=1u l=180n
Cnw84 nw84 0 2f
CT132 t132 0 0.1f
M431 t132 ni2 0 0 nch w=1u l=180n
M432 t132 ni0 0 0 nch w=1u l=180n
CT133 t133 0 0.1f
M433 t133 ni2 vdd vdd pch w=2u l=180n
M434 t132 ni0 t133 vdd pch w=2u l=180n
M435 nw85 t132 vdd vdd pch w=2u l=180n
M436 nw85 t132 0 0 nch w=1u l=180n
Cnw85 nw85 0 2f
CT134 t134 0 0.1f
CT135 t135 0 0.1f
CT136 t136 0 0.1f
M437 t134 ni8 vdd vdd pch w=2u l=180n
M438 t134 nw77 vdd vdd pch w=2u l=180n
CT137 t137 0 0.1f
M439 t134 ni8 t137 0 nch w=1u l=180n
M440 t137 nw77 0 0 nch w=1u l=180n
M441 t135 ni8 vdd vdd pch w=2u l=180n
M442 t135 t134 vdd vdd pch w=2u l=180n
CT138 t138 0 0.1f
M443 t135 ni8 t138 0 nch w=1u l=180n
M444 t138 t134 0 0 nch w=1u l=180n
M445 t136 nw77 vdd vdd pch w=2u l=180n
M446 t136 t134 vdd vdd pch w=2u l=180n
CT139 t139 0 0.1f
M447 t136 nw77 t139 0 nch w=1u l=180n
M448 t139 t134 0 0 nch w=1u l=180n
M449 nw86 t135 vdd vdd pch w=2u l=180n
M450 nw86 t136 vdd vdd pch w=2u l=180n
CT140 t140 0 0.1f
M451 nw86 t135 t140 0 nch w=1u l=180n
M452 t140 t136 0 0 nch w=1u l=180n
Cnw86 nw86 0 2f
M453 nw87 nw82 vdd vdd pch w=2u l=180n
M454 nw87 nw86 vdd vdd pch w=2u l=180n
CT141 t141 0 0.1f
M455 nw87 nw82 t141 0 nch w=1u l=180n
M456 t141 nw86 0 0 nch w=1u l=180n
Cnw87 nw87 0 2f
M457 nw88 nq0 0 0 nch w=1u l=180n
M458 nw88 nq7 0 0 nch w=1u l=180n
CT142 t142 0 0.1f
M459 t142 nq0 vdd vdd pch w=2u l=180n
M460 nw88 nq7 t142 vdd pch w=2u l=180n
Cnw88 nw88 0 2f
CT143 t143 0 0.1f
M461 t143 nq5 vdd vdd pch w=2u l=180n
M462 t143 nq15 vdd vdd pch w=2u l=180n
CT144 t144 0 0.1f
M463 t143 nq5 t144 0 nch w=1u l=180n
M464 t144 nq15 0 0 nch w=1u l=180n
M465 nw89 t143 vdd vdd pch w=2u l=180n
M466 nw89 t143 0 0 nch w=1u l=180n
Cnw89 nw89 0 2f
CT145 t145 0 0.1f
M467 t145 nq10 0 0 nch w=1u l=180n
M468 t145 ni4 0 0 nch w=1u l=180n
CT146 t146 0 0.1f
M469 t146 nq10 vdd vdd pch w=2u l=180n
M470 t145 ni4 t146 vdd pch w=2u l=180n
M471 nw90 t145 vdd vdd pch w=2u l=180n
M472 nw90 t145 0 0 nch w=1u l=180n
Cnw90 nw90 0 2f
CT147 t147 0 0.1f
CT148 t148 0 0.1f
CT149 t149 0 0.1f
M473 t147 nq15 vdd vdd pch w=2u l=180n
M474 t147 nw80 vdd vdd pch w=2u l=180n
CT150 t150 0 0.1f
M475 t147 nq15 t150 0 nch w=1u l=180n
M476 t150 nw80 0 0 nch w=1u l=180n
M477 t148 nq15 vdd vdd pch w=2u l=180n
M478 t148 t147 vdd vdd pch w=2u l=180n
CT151 t151 0 0.1f
M479 t148 nq15 t151 0 nch w=1u l=180n
M480 t151 t147 0 0 nch w=1u l=180n
M481 t149 nw80 vdd vdd pch w=2u l=180n
M482 t149 t147 vdd vdd pch w=2u l=180n
CT152 t152 0 0.1f
M483 t149 nw80 t152 0 nch w=1u l=180n
M484 t152 t147 0 0 nch w=1u l=180n
M485 nw91 t148 vdd vdd pch w=2u l=180n
M486 nw91 t149 vdd vdd pch w=2u l=180n
CT153 t153 0 0.1f
M487 nw91 t148 t153 0 nch w=1u l=180n
M488 t153 t149 0 0 nch w=1u l=180n
Cnw91 nw91 0 2f
M489 nw92 ni1 vdd vdd pch w=2u l=180n
M490 nw92 nw88 vdd vdd pch w=2u l=180n
CT154 t154 0 0.1f
M491 nw92 ni1 t154 0 nch w=1u l=180n
M492 t154 nw88 0 0 nch w=1u l=180n
Cnw92 nw92 0 2f
M493 nw93 ni6 0 0 nch w=1u l=180n
M494 nw93 nq3 0 0 nch w=1u l=180n
CT155 t155 0 0.1f
M495 t155 ni6 vdd vdd pch w=2u l=180n
M496 nw93 nq3 t155 vdd pch w=2u l=180n
Cnw93 nw93 0 2f
CT156 t156 0 0.1f
M497 t156 nw79 vdd vdd pch w=2u l=180n
M498 t156 nq10 vdd vdd pch w=2u l=180n
CT157 t157 0 0.1f
M499 t156 nw79 t157 0 nch w=1u l=180n
M500 t157 nq10 0 0 nch w=1u l=180n
M501 nw94 t156 vdd vdd pch w=2u l=180n
M502 nw94 t156 0 0 nch w=1u l=180n
Cnw94 nw94 0 2f
CT158 t158 0 0.1f
M503 t158 nw84 0 0 nch w=1u l=180n
M504 t158 nq17 0 0 nch w=1u l=180n
CT159 t159 0 0.1f
M505 t159 nw84 vdd vdd pch w=2u l=180n
M506 t158 nq17 t159 vdd pch w=2u l=180n
M507 nw95 t158 vdd vdd pch w=2u l=180n
M508 nw95 t158 0 0 nch w=1u l=180n
Cnw95 nw95 0 2f
CT160 t160 0 0.1f
CT161 t161 0 0.1f
CT162 t162 0 0.1f
M509 t160 nw89 vdd vdd pch w=2u l=180n
M510 t160 ni5 vdd vdd pch w=2u l=180n
CT163 t163 0 0.1f
M511 t160 nw89 t163 0 nch w=1u l=180n
M512 t163 ni5 0 0 nch w=1u l=180n
M513 t161 nw89 vdd vdd pch w=2u l=180n
M514 t161 t160 vdd vdd pch w=2u l=180n
CT164 t164 0 0.1f
M515 t161 nw89 t164 0 nch w=1u l=180n
M516 t164 t160 0 0 nch w=1u l=180n
M517 t162 ni5 vdd vdd pch w=2u l=180n
M518 t162 t160 vdd vdd pch w=2u l=180n
CT165 t165 0 0.1f
M519 t162 ni5 t165 0 nch w=1u l=180n
M520 t165 t160 0 0 nch w=1u l=180n
M521 nw96 t161 vdd vdd pch w=2u l=180n
M522 nw96 t162 vdd vdd pch w=2u l=180n
CT166 t166 0 0.1f
M523 nw96 t161 t166 0 nch w=1u l=180n
M524 t166 t162 0 0 nch w=1u l=180n
Cnw96 nw96 0 2f
M525 nw97 nw94 vdd vdd pch w=2u l=180n
M526 nw97 nw80 vdd vdd pch w=2u l=180n
CT167 t167 0 0.1f
M527 nw97 nw94 t167 0 nch w=1u l=180n
M528 t167 nw80 0 0 nch w=1u l=180n
Cnw97 nw97 0 2f
M529 nw98 nq1 0 0 nch w=1u l=180n
M530 nw98 nw87 0 0 nch w=1u l=180n
CT168 t168 0 0.1f
M531 t168 nq1 vdd vdd pch w=2u l=180n
M532 nw98 nw87 t168 vdd pch w=2u l=180n
Cnw98 nw98 0 2f
CT169 t169 0 0.1f
M533 t169 nq5 vdd vdd pch w=2u l=180n
M534 t169 nw94 vdd vdd pch w=2u l=180n
CT170 t170 0 0.1f
M535 t169 nq5 t170 0 nch w=1u l=180n
M536 t170 nw94 0 0 nch w=1u l=180n
M537 nw99 t169 vdd vdd pch w=2u l=180n
M538 nw99 t169 0 0 nch w=1u l=180n
Cnw99 nw99 0 2f
CT171 t171 0 0.1f
M539 t171 nq9 0 0 nch w=1u l=180n
M540 t171 nq1 0 0 nch w=1u l=180n
CT172 t172 0 0.1f
M541 t172 nq9 vdd vdd pch w=2u l=180n
M542 t171 nq1 t172 vdd pch w=2u l=180n
M543 nw100 t171 vdd vdd pch w=2u l=180n
M544 nw100 t171 0 0 nch w=1u l=180n
Cnw100 nw100 0 2f
CT173 t173 0 0.1f
CT174 t174 0 0.1f
CT175 t175 0 0.1f
M545 t173 nq13 vdd vdd pch w=2u l=180n
M546 t173 nq7 vdd vdd pch w=2u l=180n
CT176 t176 0 0.1f
M547 t173 nq13 t176 0 nch w=1u l=180n
M548 t176 nq7 0 0 nch w=1u l=180n
M549 t174 nq13 vdd vdd pch w=2u l=180n
M550 t174 t173 vdd vdd pch w=2u l=180n
CT177 t177 0 0.1f
M551 t174 nq13 t177 0 nch w=1u l=180n
M552 t177 t173 0 0 nch w=1u l=180n
M553 t175 nq7 vdd vdd pch w=2u l=180n
M554 t175 t173 vdd vdd pch w=2u l=180n
CT178 t178 0 0.1f
M555 t175 nq7 t178 0 nch w=1u l=180n
M556 t178 t173 0 0 nch w=1u l=180n
M557 nw101 t174 vdd vdd pch w=2u l=180n
M558 nw101 t175 vdd vdd pch w=2u l=180n
CT179 t179 0 0.1f
M559 nw101 t174 t179 0 nch w=1u l=180n
M560 t179 t175 0 0 nch w=1u l=180n
Cnw101 nw101 0 2f
M561 nw102 nq17 vdd vdd pch w=2u l=180n
M562 nw102 nq13 vdd vdd pch w=2u l=180n
CT180 t180 0 0.1f
M563 nw102 nq17 t180 0 nch w=1u l=180n
M564 t180 nq13 0 0 nch w=1u l=180n
Cnw102 nw102 0 2f
M565 nw103 ni2 0 0 nch w=1u l=180n
M566 nw103 ni0 0 0 nch w=1u l=180n
CT181 t181 0 0.1f
M567 t181 ni2 vdd vdd pch w=2u l=180n
M568 nw103 ni0 t181 vdd pch w=2u l=180n
Cnw103 nw103 0 2f
CT182 t182 0 0.1f
M569 t182 ni6 vdd vdd pch w=2u l=180n
M570 t182 ni7 vdd vdd pch w=2u l=180n
CT183 t183 0 0.1f
M571 t182 ni6 t183 0 nch w=1u l=180n
M572 t183 ni7 0 0 nch w=1u l=180n
M573 nw104 t182 vdd vdd pch w=2u l=180n
M574 nw104 t182 0 0 nch w=1u l=180n
Cnw104 nw104 0 2f
CT184 t184 0 0.1f
M575 t184 nw78 0 0 nch w=1u l=180n
M576 t184 nw80 0 0 nch w=1u l=180n
CT185 t185 0 0.1f
M577 t185 nw78 vdd vdd pch w=2u l=180n
M578 t184 nw80 t185 vdd pch w=2u l=180n
M579 nw105 t184 vdd vdd pch w=2u l=180n
M580 nw105 t184 0 0 nch w=1u l=180n
Cnw105 nw105 0 2f
CT186 t186 0 0.1f
CT187 t187 0 0.1f
CT188 t188 0 0.1f
M581 t186 nw82 vdd vdd pch w=2u l=180n
M582 t186 nw86 vdd vdd pch w=2u l=180n
CT189 t189 0 0.1f
M583 t186 nw82 t189 0 nch w=1u l=180n
M584 t189 nw86 0 0 nch w=1u l=180n
M585 t187 nw82 vdd vdd pch w=2u l=180n
M586 t187 t186 vdd vdd pch w=2u l=180n
CT190 t190 0 0.1f
M587 t187 nw82 t190 0 nch w=1u l=180n
M588 t190 t186 0 0 nch w=1u l=180n
M589 t188 nw86 vdd vdd pch w=2u l=180n
M590 t188 t186 vdd vdd pch w=2u l=180n
CT191 t191 0 0.1f
M591 t188 nw86 t191 0 nch w=1u l=180n
M592 t191 t186 0 0 nch w=1u l=180n
M593 nw106 t187 vdd vdd pch w=2u l=180n
M594 nw106 t188 vdd vdd pch w=2u l=180n
CT192 t192 0 0.1f
M595 nw106 t187 t192 0 nch w=1u l=180n
M596 t192 t188 0 0 nch w=1u l=180n
Cnw106 nw106 0 2f
M597 nw107 nw86 vdd vdd pch w=2u l=180n
M598 nw107 nw92 vdd vdd pch w=2u l=180n
CT193 t193 0 0.1f
M599 nw107 nw86 t193 0 nch w=1u l=180n
M600 t193 nw92 0 0 nch w=1u l=180n
Cnw107 nw107 0 2f
M601 nw108 nw90 0 0 nch w=1u l=180n
M602 nw108 nw98 0 0 nch w=1u l=180n
CT194 t194 0 0.1f
M603 t194 nw90 vdd vdd pch w=2u l=180n
M604 nw108 nw98 t194 vdd pch w=2u l=180n
Cnw108 nw108 0 2f
CT195 t195 0 0.1f
M605 t195 nw94 vdd vdd pch w=2u l=180n
M606 t195 nw104 vdd vdd pch w=2u l=180n
CT196 t196 0 0.1f
M607 t195 nw94 t196 0 nch w=1u l=180n
M608 t196 nw104 0 0 nch w=1u l=180n
M609 nw109 t195 vdd vdd pch w=2u l=180n
M610 nw109 t195 0 0 nch w=1u l=180n
Cnw109 nw109 0 2f
CT197 t197 0 0.1f
M611 t197 nw98 0 0 nch w=1u l=180n
M612 t197 nq0 0 0 nch w=1u l=180n
CT198 t198 0 0.1f
M613 t198 nw98 vdd vdd pch w=2u l=180n
M614 t197 nq0 t198 vdd pch w=2u l=180n
M615 nw110 t197 vdd vdd pch w=2u l=180n
M616 nw110 t197 0 0 nch w=1u l=180n
Cnw110 nw110 0 2f
CT199 t199 0 0.1f
CT200 t200 0 0.1f
CT201 t201 0 0.1f
M617 t199 nw102 vdd vdd pch w=2u l=180n
M618 t199 nq5 vdd vdd pch w=2u l=180n
CT202 t202 0 0.1f
M619 t199 nw102 t202 0 nch w=1u l=180n
M620 t202 nq5 0 0 nch w=1u l=180n
M621 t200 nw102 vdd vdd pch w=2u l=180n
M622 t200 t199 vdd vdd pch w=2u l=180n
CT203 t203 0 0.1f
M623 t200 nw102 t203 0 nch w=1u l=180n
M624 t203 t199 0 0 nch w=1u l=180n
M625 t201 nq5 vdd vdd pch w=2u l=180n
M626 t201 t199 vdd vdd pch w=2u l=180n
CT204 t204 0 0.1f
M627 t201 nq5 t204 0 nch w=1u l=180n
M628 t204 t199 0 0 nch w=1u l=180n
M629 nw111 t200 vdd vdd pch w=2u l=180n
M630 nw111 t201 vdd vdd pch w=2u l=180n
CT205 t205 0 0.1f
M631 nw111 t200 t205 0 nch w=1u l=180n
M632 t205 t201 0 0 nch w=1u l=180n
Cnw111 nw111 0 2f
M633 nw112 nw106 vdd vdd pch w=2u l=180n
M634 nw112 nq10 vdd vdd pch w=2u l=180n
CT206 t206 0 0.1f
M635 nw112 nw106 t206 0 nch w=1u l=180n
M636 t206 nq10 0 0 nch w=1u l=180n
Cnw112 nw112 0 2f
M637 nw113 nw110 0 0 nch w=1u l=180n
M638 nw113 nq15 0 0 nch w=1u l=180n
CT207 t207 0 0.1f
M639 t207 nw110 vdd vdd pch w=2u l=180n
M640 nw113 nq15 t207 vdd pch w=2u l=180n
Cnw113 nw113 0 2f
CT208 t208 0 0.1f
M641 t208 nq0 vdd vdd pch w=2u l=180n
M642 t208 ni1 vdd vdd pch w=2u l=180n
CT209 t209 0 0.1f
M643 t208 nq0 t209 0 nch w=1u l=180n
M644 t209 ni1 0 0 nch w=1u l=180n
M645 nw114 t208 vdd vdd pch w=2u l=180n
M646 nw114 t208 0 0 nch w=1u l=180n
Cnw114 nw114 0 2f
CT210 t210 0 0.1f
M647 t210 nq3 0 0 nch w=1u l=180n
M648 t210 ni6 0 0 nch w=1u l=180n
CT211 t211 0 0.1f
M649 t211 nq3 vdd vdd pch w=2u l=180n
M650 t210 ni6 t211 vdd pch w=2u l=180n
M651 nw115 t210 vdd vdd pch w=2u l=180n
M652 nw115 t210 0 0 nch w=1u l=180n
Cnw115 nw115 0 2f
CT212 t212 0 0.1f
CT213 t213 0 0.1f
CT214 t214 0 0.1f
M653 t212 nq6 vdd vdd pch w=2u l=180n
M654 t212 nw79 vdd vdd pch w=2u l=180n
CT215 t215 0 0.1f
M655 t212 nq6 t215 0 nch w=1u l=180n
M656 t215 nw79 0 0 nch w=1u l=180n
M657 t213 nq6 vdd vdd pch w=2u l=180n
M658 t213 t212 vdd vdd pch w=2u l=180n
CT216 t216 0 0.1f
M659 t213 nq6 t216 0 nch w=1u l=180n
M660 t216 t212 0 0 nch w=1u l=180n
M661 t214 nw79 vdd vdd pch w=2u l=180n
M662 t214 t212 vdd vdd pch w=2u l=180n
CT217 t217 0 0.1f
M663 t214 nw79 t217 0 nch w=1u l=180n
M664 t217 t212 0 0 nch w=1u l=180n
M665 nw116 t213 vdd vdd pch w=2u l=180n
M666 nw116 t214 vdd vdd pch w=2u l=180n
CT218 t218 0 0.1f
M667 nw116 t213 t218 0 nch w=1u l=180n
M668 t218 t214 0 0 nch w=1u l=180n
Cnw116 nw116 0 2f
M669 nw117 nq9 vdd vdd pch w=2u l=180n
M670 nw117 nw84 vdd vdd pch w=2u l=180n
CT219 t219 0 0.1f
M671 nw117 nq9 t219 0 nch w=1u l=180n
M672 t219 nw84 0 0 nch w=1u l=180n
Cnw117 nw117 0 2f
M673 nw118 nq12 0 0 nch w=1u l=180n
M674 nw118 nw89 0 0 nch w=1u l=180n
CT220 t220 0 0.1f
M675 t220 nq12 vdd vdd pch w=2u l=180n
M676 nw118 nw89 t220 vdd pch w=2u l=180n
Cnw118 nw118 0 2f
CT221 t221 0 0.1f
M677 t221 nq15 vdd vdd pch w=2u l=180n
M678 t221 nw94 vdd vdd pch w=2u l=180n
CT222 t222 0 0.1f
M679 t221 nq15 t222 0 nch w=1u l=180n
M680 t222 nw94 0 0 nch w=1u l=180n
M681 nw119 t221 vdd vdd pch w=2u l=180n
M682 nw119 t221 0 0 nch w=1u l=180n
Cnw119 nw119 0 2f
CT223 t223 0 0.1f
M683 t223 nq18 0 0 nch w=1u l=180n
M684 t223 nw99 0 0 nch w=1u l=180n
CT224 t224 0 0.1f
M685 t224 nq18 vdd vdd pch w=2u l=180n
M686 t223 nw99 t224 vdd pch w=2u l=180n
M687 nw120 t223 vdd vdd pch w=2u l=180n
M688 nw120 t223 0 0 nch w=1u l=180n
Cnw120 nw120 0 2f
CT225 t225 0 0.1f
CT226 t226 0 0.1f
CT227 t227 0 0.1f
M689 t225 ni2 vdd vdd pch w=2u l=180n
M690 t225 nw104 vdd vdd pch w=2u l=180n
CT228 t228 0 0.1f
M691 t225 ni2 t228 0 nch w=1u l=180n
M692 t228 nw104 0 0 nch w=1u l=180n
M693 t226 ni2 vdd vdd pch w=2u l=180n
M694 t226 t225 vdd vdd pch w=2u l=180n
CT229 t229 0 0.1f
M695 t226 ni2 t229 0 nch w=1u l=180n
M696 t229 t225 0 0 nch w=1u l=180n
M697 t227 nw104 vdd vdd pch w=2u l=180n
M698 t227 t225 vdd vdd pch w=2u l=180n
CT230 t230 0 0.1f
M699 t227 nw104 t230 0 nch w=1u l=180n
M700 t230 t225 0 0 nch w=1u l=180n
M701 nw121 t226 vdd vdd pch w=2u l=180n
M702 nw121 t227 vdd vdd pch w=2u l=180n
CT231 t231 0 0.1f
M703 nw121 t226 t231 0 nch w=1u l=180n
M704 t231 t227 0 0 nch w=1u l=180n
Cnw121 nw121 0 2f
M705 nw122 ni5 vdd vdd pch w=2u l=180n
M706 nw122 nw109 vdd vdd pch w=2u l=180n
CT232 t232 0 0.1f
M707 nw122 ni5 t232 0 nch w=1u l=180n
M708 t232 nw109 0 0 nch w=1u l=180n
Cnw122 nw122 0 2f
M709 nw123 ni8 0 0 nch w=1u l=180n
M710 nw123 nw114 0 0 nch w=1u l=180n
CT233 t233 0 0.1f
M711 t233 ni8 vdd vdd pch w=2u l=180n
M712 nw123 nw114 t233 vdd pch w=2u l=180n
Cnw123 nw123 0 2f
CT234 t234 0 0.1f
M713 t234 nw79 vdd vdd pch w=2u l=180n
M714 t234 nw119 vdd vdd pch w=2u l=180n
CT235 t235 0 0.1f
M715 t234 nw79 t235 0 nch w=1u l=180n
M716 t235 nw119 0 0 nch w=1u l=180n
M717 nw124 t234 vdd vdd pch w=2u l=180n
M718 nw124 t234 0 0 nch w=1u l=180n
Cnw124 nw124 0 2f
CT236 t236 0 0.1f
M719 t236 nw82 0 0 nch w=1u l=180n
M720 t236 nw124 0 0 nch w=1u l=180n
CT237 t237 0 0.1f
M721 t237 nw82 vdd vdd pch w=2u l=180n
M722 t236 nw124 t237 vdd pch w=2u l=180n
M723 nw125 t236 vdd vdd pch w=2u l=180n
M724 nw125 t236 0 0 nch w=1u l=180n
Cnw125 nw125 0 2f
CT238 t238 0 0.1f
CT239 t239 0 0.1f
CT240 t240 0 0.1f
M725 t238 nw85 vdd vdd pch w=2u l=180n
M726 t238 nq3 vdd vdd pch w=2u l=180n
CT241 t241 0 0.1f
M727 t238 nw85 t241 0 nch w=1u l=180n
M728 t241 nq3 0 0 nch w=1u l=180n
M729 t239 nw85 vdd vdd pch w=2u l=180n
M730 t239 t238 vdd vdd pch w=2u l=180n
CT242 t242 0 0.1f
M731 t239 nw85 t242 0 nch w=1u l=180n
M732 t242 t238 0 0 nch w=1u l=180n
M733 t240 nq3 vdd vdd pch w=2u l=180n
M734 t240 t238 vdd vdd pch w=2u l=180n
CT243 t243 0 0.1f
M735 t240 nq3 t243 0 nch w=1u l=180n
M736 t243 t238 0 0 nch w=1u l=180n
M737 nw126 t239 vdd vdd pch w=2u l=180n
M738 nw126 t240 vdd vdd pch w=2u l=180n
CT244 t244 0 0.1f
M739 nw126 t239 t244 0 nch w=1u l=180n
M740 t244 t240 0 0 nch w=1u l=180n
Cnw126 nw126 0 2f
M741 nw127 nw88 vdd vdd pch w=2u l=180n
M742 nw127 nq7 vdd vdd pch w=2u l=180n
CT245 t245 0 0.1f
M743 nw127 nw88 t245 0 nch w=1u l=180n
M744 t245 nq7 0 0 nch w=1u l=180n
Cnw127 nw127 0 2f
M745 nw128 nw91 0 0 nch w=1u l=180n
M746 nw128 nq11 0 0 nch w=1u l=180n
CT246 t246 0 0.1f
M747 t246 nw91 vdd vdd pch w=2u l=180n
M748 nw128 nq11 t246 vdd pch w=2u l=180n
Cnw128 nw128 0 2f
CT247 t247 0 0.1f
M749 t247 nw94 vdd vdd pch w=2u l=180n
M750 t247 nq15 vdd vdd pch w=2u l=180n
CT248 t248 0 0.1f
M751 t247 nw94 t248 0 nch w=1u l=180n
M752 t248 nq15 0 0 nch w=1u l=180n
M753 nw129 t247 vdd vdd pch w=2u l=180n
M754 nw129 t247 0 0 nch w=1u l=180n
Cnw129 nw129 0 2f
CT249 t249 0 0.1f
M755 t249 nw97 0 0 nch w=1u l=180n
M756 t249 ni0 0 0 nch w=1u l=180n
CT250 t250 0 0.1f
M757 t250 nw97 vdd vdd pch w=2u l=180n
M758 t249 ni0 t250 vdd pch w=2u l=180n
M759 nw130 t249 vdd vdd pch w=2u l=180n
M760 nw130 t249 0 0 nch w=1u l=180n
Cnw130 nw130 0 2f
CT251 t251 0 0.1f
CT252 t252 0 0.1f
CT253 t253 0 0.1f
M761 t251 nw100 vdd vdd pch w=2u l=180n
M762 t251 ni4 vdd vdd pch w=2u l=180n
CT254 t254 0 0.1f
M763 t251 nw100 t254 0 nch w=1u l=180n
M764 t254 ni4 0 0 nch w=1u l=180n
M765 t252 nw100 vdd vdd pch w=2u l=180n
M766 t252 t251 vdd vdd pch w=2u l=180n
CT255 t255 0 0.1f
M767 t252 nw100 t255 0 nch w=1u l=180n
M768 t255 t251 0 0 nch w=1u l=180n
M769 t253 ni4 vdd vdd pch w=2u l=180n
M770 t253 t251 vdd vdd pch w=2u l=180n
CT256 t256 0 0.1f
M771 t253 ni4 t256 0 nch w=1u l=180n
M772 t256 t251 0 0 nch w=1u l=180n
M773 nw131 t252 vdd vdd pch w=2u l=180n
M774 nw131 t253 vdd vdd pch w=2u l=180n
CT257 t257 0 0.1f
M775 nw131 t252 t257 0 nch w=1u l=180n
M776 t257 t253 0 0 nch w=1u l=180n
Cnw131 nw131 0 2f
M777 nw132 nw103 vdd vdd pch w=2u l=180n
M778 nw132 ni8 vdd vdd pch w=2u l=180n
CT258 t258 0 0.1f
M779 nw132 nw103 t258 0 nch w=1u l=180n
M780 t258 ni8 0 0 nch w=1u l=180n
Cnw132 nw132 0 2f
M781 nw133 nw106 0 0 nch w=1u l=180n
M782 nw133 nw80 0 0 nch w=1u l=180n
CT259 t259 0 0.1f
M783 t259 nw106 vdd vdd pch w=2u l=180n
M784 nw133 nw80 t259 vdd pch w=2u l=180n
Cnw133 nw133 0 2f
CT260 t260 0 0.1f
M785 t260 nw109 vdd vdd pch w=2u l=180n
M786 t260 nw84 vdd vdd pch w=2u l=180n
CT261 t261 0 0.1f
M787 t260 nw109 t261 0 nch w=1u l=180n
M788 t261 nw84 0 0 nch w=1u l=180n
M789 nw134 t260 vdd vdd pch w=2u l=180n
M790 nw134 t260 0 0 nch w=1u l=180n
Cnw134 nw134 0 2f
CT262 t262 0 0.1f
M791 t262 nw112 0 0 nch w=1u l=180n
M792 t262 nw88 0 0 nch w=1u l=180n
CT263 t263 0 0.1f
M793 t263 nw112 vdd vdd pch w=2u l=180n
M794 t262 nw88 t263 vdd pch w=2u l=180n
M795 nw135 t262 vdd vdd pch w=2u l=180n
M796 nw135 t262 0 0 nch w=1u l=180n
Cnw135 nw135 0 2f
CT264 t264 0 0.1f
CT265 t265 0 0.1f
CT266 t266 0 0.1f
M797 t264 nw115 vdd vdd pch w=2u l=180n
M798 t264 nw92 vdd vdd pch w=2u l=180n
CT267 t267 0 0.1f
M799 t264 nw115 t267 0 nch w=1u l=180n
M800 t267 nw92 0 0 nch w=1u l=180n
M801 t265 nw115 vdd vdd pch w=2u l=180n
M802 t265 t264 vdd vdd pch w=2u l=180n
CT268 t268 0 0.1f
M803 t265 nw115 t268 0 nch w=1u l=180n
M804 t268 t264 0 0 nch w=1u l=180n
M805 t266 nw92 vdd vdd pch w=2u l=180n
M806 t266 t264 vdd vdd pch w=2u l=180n
CT269 t269 0 0.1f
M807 t266 nw92 t269 0 nch w=1u l=180n
M808 t269 t264 0 0 nch w=1u l=180n
M809 nw136 t265 vdd vdd pch w=2u l=180n
M810 nw136 t266 vdd vdd pch w=2u l=180n
CT270 t270 0 0.1f
M811 nw136 t265 t270 0 nch w=1u l=180n
M812 t270 t266 0 0 nch w=1u l=180n
Cnw136 nw136 0 2f
M813 nw137 nw118 vdd vdd pch w=2u l=180n
M814 nw137 nw96 vdd vdd pch w=2u l=180n
CT271 t271 0 0.1f
M815 nw137 nw118 t271 0 nch w=1u l=180n
M816 t271 nw96 0 0 nch w=1u l=180n
Cnw137 nw137 0 2f
M817 nw138 nw121 0 0 nch w=1u l=180n
M818 nw138 nw100 0 0 nch w=1u l=180n
CT272 t272 0 0.1f
M819 t272 nw121 vdd vdd pch w=2u l=180n
M820 nw138 nw100 t272 vdd pch w=2u l=180n
Cnw138 nw138 0 2f
CT273 t273 0 0.1f
M821 t273 nw124 vdd vdd pch w=2u l=180n
M822 t273 nw104 vdd vdd pch w=2u l=180n
CT274 t274 0 0.1f
M823 t273 nw124 t274 0 nch w=1u l=180n
M824 t274 nw104 0 0 nch w=1u l=180n
M825 nw139 t273 vdd vdd pch w=2u l=180n
M826 nw139 t273 0 0 nch w=1u l=180n
Cnw139 nw139 0 2f
CT275 t275 0 0.1f
M827 t275 nw127 0 0 nch w=1u l=180n
M828 t275 nw108 0 0 nch w=1u l=180n
CT276 t276 0 0.1f
M829 t276 nw127 vdd vdd pch w=2u l=180n
M830 t275 nw108 t276 vdd pch w=2u l=180n
M831 nw140 t275 vdd vdd pch w=2u l=180n
M832 nw140 t275 0 0 nch w=1u l=180n
Cnw140 nw140 0 2f
CT277 t277 0 0.1f
CT278 t278 0 0.1f
CT279 t279 0 0.1f
M833 t277 nw130 vdd vdd pch w=2u l=180n
M834 t277 nw112 vdd vdd pch w=2u l=180n
CT280 t280 0 0.1f
M835 t277 nw130 t280 0 nch w=1u l=180n
M836 t280 nw112 0 0 nch w=1u l=180n
M837 t278 nw130 vdd vdd pch w=2u l=180n
M838 t278 t277 vdd vdd pch w=2u l=180n
CT281 t281 0 0.1f
M839 t278 nw130 t281 0 nch w=1u l=180n
M840 t281 t277 0 0 nch w=1u l=180n
M841 t279 nw112 vdd vdd pch w=2u l=180n
M842 t279 t277 vdd vdd pch w=2u l=180n
CT282 t282 0 0.1f
M843 t279 nw112 t282 0 nch w=1u l=180n
M844 t282 t277 0 0 nch w=1u l=180n
M845 nw141 t278 vdd vdd pch w=2u l=180n
M846 nw141 t279 vdd vdd pch w=2u l=180n
CT283 t283 0 0.1f
M847 nw141 t278 t283 0 nch w=1u l=180n
M848 t283 t279 0 0 nch w=1u l=180n
Cnw141 nw141 0 2f
M849 nw142 nw133 vdd vdd pch w=2u l=180n
M850 nw142 nw116 vdd vdd pch w=2u l=180n
CT284 t284 0 0.1f
M851 nw142 nw133 t284 0 nch w=1u l=180n
M852 t284 nw116 0 0 nch w=1u l=180n
Cnw142 nw142 0 2f
M853 nw143 nw136 0 0 nch w=1u l=180n
M854 nw143 nw120 0 0 nch w=1u l=180n
CT285 t285 0 0.1f
M855 t285 nw136 vdd vdd pch w=2u l=180n
M856 nw143 nw120 t285 vdd pch w=2u l=180n
Cnw143 nw143 0 2f
CT286 t286 0 0.1f
M857 t286 nw139 vdd vdd pch w=2u l=180n
M858 t286 nw124 vdd vdd pch w=2u l=180n
CT287 t287 0 0.1f
M859 t286 nw139 t287 0 nch w=1u l=180n
M860 t287 nw124 0 0 nch w=1u l=180n
M861 nw144 t286 vdd vdd pch w=2u l=180n
M862 nw144 t286 0 0 nch w=1u l=180n
Cnw144 nw144 0 2f
CT288 t288 0 0.1f
M863 t288 nw142 0 0 nch w=1u l=180n
M864 t288 nw128 0 0 nch w=1u l=180n
CT289 t289 0 0.1f
M865 t289 nw142 vdd vdd pch w=2u l=180n
M866 t288 nw128 t289 vdd pch w=2u l=180n
M867 nw145 t288 vdd vdd pch w=2u l=180n
M868 nw145 t288 0 0 nch w=1u l=180n
Cnw145 nw145 0 2f
CT290 t290 0 0.1f
CT291 t291 0 0.1f
CT292 t292 0 0.1f
M869 t290 nw145 vdd vdd pch w=2u l=180n
M870 t290 nw132 vdd vdd pch w=2u l=180n
CT293 t293 0 0.1f
M871 t290 nw145 t293 0 nch w=1u l=180n
M872 t293 nw132 0 0 nch w=1u l=180n
M873 t291 nw145 vdd vdd pch w=2u l=180n
M874 t291 t290 vdd vdd pch w=2u l=180n
CT294 t294 0 0.1f
M875 t291 nw145 t294 0 nch w=1u l=180n
M876 t294 t290 0 0 nch w=1u l=180n
M877 t292 nw132 vdd vdd pch w=2u l=180n
M878 t292 t290 vdd vdd pch w=2u l=180n
CT295 t295 0 0.1f
M879 t292 nw132 t295 0 nch w=1u l=180n
M880 t295 t290 0 0 nch w=1u l=180n
M881 nw146 t291 vdd vdd pch w=2u l=180n
M882 nw146 t292 vdd vdd pch w=2u l=180n
CT296 t296 0 0.1f
M883 nw146 t291 t296 0 nch w=1u l=180n
M884 t296 t292 0 0 nch w=1u l=180n
Cnw146 nw146 0 2f
M885 nw147 nq1 vdd vdd pch w=2u l=180n
M886 nw147 nw136 vdd vdd pch w=2u l=180n
CT297 t297 0 0.1f
M887 nw147 nq1 t297 0 nch w=1u l=180n
M888 t297 nw136 0 0 nch w=1u l=180n
Cnw147 nw147 0 2f
M889 nw148 nq3 0 0 nch w=1u l=180n
M890 nw148 nw140 0 0 nch w=1u l=180n
CT298 t298 0 0.1f
M891 t298 nq3 vdd vdd pch w=2u l=180n
M892 nw148 nw140 t298 vdd pch w=2u l=180n
Cnw148 nw148 0 2f
CT299 t299 0 0.1f
M893 t299 nq5 vdd vdd pch w=2u l=180n
M894 t299 nw144 vdd vdd pch w=2u l=180n
CT300 t300 0 0.1f
M895 t299 nq5 t300 0 nch w=1u l=180n
M896 t300 nw144 0 0 nch w=1u l=180n
M897 nw149 t299 vdd vdd pch w=2u l=180n
M898 nw149 t299 0 0 nch w=1u l=180n
Cnw149 nw149 0 2f
CT301 t301 0 0.1f
M899 t301 nq7 0 0 nch w=1u l=180n
M900 t301 nw148 0 0 nch w=1u l=180n
CT302 t302 0 0.1f
M901 t302 nq7 vdd vdd pch w=2u l=180n
M902 t301 nw148 t302 vdd pch w=2u l=180n
M903 nw150 t301 vdd vdd pch w=2u l=180n
M904 nw150 t301 0 0 nch w=1u l=180n
Cnw150 nw150 0 2f
CT303 t303 0 0.1f
CT304 t304 0 0.1f
CT305 t305 0 0.1f
M905 t303 nq9 vdd vdd pch w=2u l=180n
M906 t303 nq1 vdd vdd pch w=2u l=180n
CT306 t306 0 0.1f
M907 t303 nq9 t306 0 nch w=1u l=180n
M908 t306 nq1 0 0 nch w=1u l=180n
M909 t304 nq9 vdd vdd pch w=2u l=180n
M910 t304 t303 vdd vdd pch w=2u l=180n
CT307 t307 0 0.1f
M911 t304 nq9 t307 0 nch w=1u l=180n
M912 t307 t303 0 0 nch w=1u l=180n
M913 t305 nq1 vdd vdd pch w=2u l=180n
M914 t305 t303 vdd vdd pch w=2u l=180n
CT308 t308 0 0.1f
M915 t305 nq1 t308 0 nch w=1u l=180n
M916 t308 t303 0 0 nch w=1u l=180n
M917 nw151 t304 vdd vdd pch w=2u l=180n
M918 nw151 t305 vdd vdd pch w=2u l=180n
CT309 t309 0 0.1f
M919 nw151 t304 t309 0 nch w=1u l=180n
M920 t309 t305 0 0 nch w=1u l=180n
Cnw151 nw151 0 2f
M921 nw152 nq11 vdd vdd pch w=2u l=180n
M922 nw152 nq4 vdd vdd pch w=2u l=180n
CT310 t310 0 0.1f
M923 nw152 nq11 t310 0 nch w=1u l=180n
M924 t310 nq4 0 0 nch w=1u l=180n
Cnw152 nw152 0 2f
M925 nw153 nq13 0 0 nch w=1u l=180n
M926 nw153 nq7 0 0 nch w=1u l=180n
CT311 t311 0 0.1f
M927 t311 nq13 vdd vdd pch w=2u l=180n
M928 nw153 nq7 t311 vdd pch w=2u l=180n
Cnw153 nw153 0 2f
CT312 t312 0 0.1f
M929 t312 nq15 vdd vdd pch w=2u l=180n
M930 t312 nq10 vdd vdd pch w=2u l=180n
CT313 t313 0 0.1f
M931 t312 nq15 t313 0 nch w=1u l=180n
M932 t313 nq10 0 0 nch w=1u l=180n
M933 nw154 t312 vdd vdd pch w=2u l=180n
M934 nw154 t312 0 0 nch w=1u l=180n
Cnw154 nw154 0 2f
CT314 t314 0 0.1f
M935 t314 nq17 0 0 nch w=1u l=180n
M936 t314 nq13 0 0 nch w=1u l=180n
CT315 t315 0 0.1f
M937 t315 nq17 vdd vdd pch w=2u l=180n
M938 t314 nq13 t315 vdd pch w=2u l=180n
M939 nw155 t314 vdd vdd pch w=2u l=180n
M940 nw155 t314 0 0 nch w=1u l=180n
Cnw155 nw155 0 2f
CT316 t316 0 0.1f
CT317 t317 0 0.1f
CT318 t318 0 0.1f
M941 t316 ni0 vdd vdd pch w=2u l=180n
M942 t316 nq16 vdd vdd pch w=2u l=180n
CT319 t319 0 0.1f
M943 t316 ni0 t319 0 nch w=1u l=180n
M944 t319 nq16 0 0 nch w=1u l=180n
M945 t317 ni0 vdd vdd pch w=2u l=180n
M946 t317 t316 vdd vdd pch w=2u l=180n
CT320 t320 0 0.1f
M947 t317 ni0 t320 0 nch w=1u l=180n
M948 t320 t316 0 0 nch w=1u l=180n
M949 t318 nq16 vdd vdd pch w=2u l=180n
M950 t318 t316 vdd vdd pch w=2u l=180n
CT321 t321 0 0.1f
M951 t318 nq16 t321 0 nch w=1u l=180n
M952 t321 t316 0 0 nch w=1u l=180n
M953 nw156 t317 vdd vdd pch w=2u l=180n
M954 nw156 t318 vdd vdd pch w=2u l=180n
CT322 t322 0 0.1f
M955 nw156 t317 t322 0 nch w=1u l=180n
M956 t322 t318 0 0 nch w=1u l=180n
Cnw156 nw156 0 2f
M957 nw157 ni2 vdd vdd pch w=2u l=180n
M958 nw157 ni0 vdd vdd pch w=2u l=180n
CT323 t323 0 0.1f
M959 nw157 ni2 t323 0 nch w=1u l=180n
M960 t323 ni0 0 0 nch w=1u l=180n
Cnw157 nw157 0 2f
M961 nw158 ni4 0 0 nch w=1u l=180n
M962 nw158 ni3 0 0 nch w=1u l=180n
CT324 t324 0 0.1f
M963 t324 ni4 vdd vdd pch w=2u l=180n
M964 nw158 ni3 t324 vdd pch w=2u l=180n
Cnw158 nw158 0 2f
CT325 t325 0 0.1f
M965 t325 ni6 vdd vdd pch w=2u l=180n
M966 t325 nw130 vdd vdd pch w=2u l=180n
CT326 t326 0 0.1f
M967 t325 ni6 t326 0 nch w=1u l=180n
M968 t326 nw130 0 0 nch w=1u l=180n
M969 nw159 t325 vdd vdd pch w=2u l=180n
M970 nw159 t325 0 0 nch w=1u l=180n
Cnw159 nw159 0 2f
CT327 t327 0 0.1f
M971 t327 ni8 0 0 nch w=1u l=180n
M972 t327 nw77 0 0 nch w=1u l=180n
CT328 t328 0 0.1f
M973 t328 ni8 vdd vdd pch w=2u l=180n
M974 t327 nw77 t328 vdd pch w=2u l=180n
M975 nw160 t327 vdd vdd pch w=2u l=180n
M976 nw160 t327 0 0 nch w=1u l=180n
Cnw160 nw160 0 2f
CT329 t329 0 0.1f
CT330 t330 0 0.1f
CT331 t331 0 0.1f
M977 t329 nw78 vdd vdd pch w=2u l=180n
M978 t329 nw80 vdd vdd pch w=2u l=180n
CT332 t332 0 0.1f
M979 t329 nw78 t332 0 nch w=1u l=180n
M980 t332 nw80 0 0 nch w=1u l=180n
M981 t330 nw78 vdd vdd pch w=2u l=180n
M982 t330 t329 vdd vdd pch w=2u l=180n
CT333 t333 0 0.1f
M983 t330 nw78 t333 0 nch w=1u l=180n
M984 t333 t329 0 0 nch w=1u l=180n
M985 t331 nw80 vdd vdd pch w=2u l=180n
M986 t331 t329 vdd vdd pch w=2u l=180n
CT334 t334 0 0.1f
M987 t331 nw80 t334 0 nch w=1u l=180n
M988 t334 t329 0 0 nch w=1u l=180n
M989 nw161 t330 vdd vdd pch w=2u l=180n
M990 nw161 t331 vdd vdd pch w=2u l=180n
CT335 t335 0 0.1f
M991 nw161 t330 t335 0 nch w=1u l=180n
M992 t335 t331 0 0 nch w=1u l=180n
Cnw161 nw161 0 2f
M993 nw162 nw80 vdd vdd pch w=2u l=180n
M994 nw162 nw83 vdd vdd pch w=2u l=180n
CT336 t336 0 0.1f
M995 nw162 nw80 t336 0 nch w=1u l=180n
M996 t336 nw83 0 0 nch w=1u l=180n
Cnw162 nw162 0 2f
M997 nw163 nw82 0 0 nch w=1u l=180n
M998 nw163 nw86 0 0 nch w=1u l=180n
CT337 t337 0 0.1f
M999 t337 nw82 vdd vdd pch w=2u l=180n
M1000 nw163 nw86 t337 vdd pch w=2u l=180n
Cnw163 nw163 0 2f
CT338 t338 0 0.1f
M1001 t338 nw84 vdd vdd pch w=2u l=180n
M1002 t338 nw89 vdd vdd pch w=2u l=180n
CT339 t339 0 0.1f
M1003 t338 nw84 t339 0 nch w=1u l=180n
M1004 t339 nw89 0 0 nch w=1u l=180n
M1005 nw164 t338 vdd vdd pch w=2u l=180n
M1006 nw164 t338 0 0 nch w=1u l=180n
Cnw164 nw164 0 2f
CT340 t340 0 0.1f
M1007 t340 nw86 0 0 nch w=1u l=180n
M1008 t340 nw92 0 0 nch w=1u l=180n
CT341 t341 0 0.1f
M1009 t341 nw86 vdd vdd pch w=2u l=180n
M1010 t340 nw92 t341 vdd pch w=2u l=180n
M1011 nw165 t340 vdd vdd pch w=2u l=180n
M1012 nw165 t340 0 0 nch w=1u l=180n
Cnw165 nw165 0 2f
CT342 t342 0 0.1f
CT343 t343 0 0.1f
CT344 t344 0 0.1f
M1013 t342 nw88 vdd vdd pch w=2u l=180n
M1014 t342 nw95 vdd vdd pch w=2u l=180n
CT345 t345 0 0.1f
M1015 t342 nw88 t345 0 nch w=1u l=180n
M1016 t345 nw95 0 0 nch w=1u l=180n
M1017 t343 nw88 vdd vdd pch w=2u l=180n
M1018 t343 t342 vdd vdd pch w=2u l=180n
CT346 t346 0 0.1f
M1019 t343 nw88 t346 0 nch w=1u l=180n
M1020 t346 t342 0 0 nch w=1u l=180n
M1021 t344 nw95 vdd vdd pch w=2u l=180n
M1022 t344 t342 vdd vdd pch w=2u l=180n
CT347 t347 0 0.1f
M1023 t344 nw95 t347 0 nch w=1u l=180n
M1024 t347 t342 0 0 nch w=1u l=180n
M1025 nw166 t343 vdd vdd pch w=2u l=180n
M1026 nw166 t344 vdd vdd pch w=2u l=180n
CT348 t348 0 0.1f
M1027 nw166 t343 t348 0 nch w=1u l=180n
M1028 t348 t344 0 0 nch w=1u l=180n
Cnw166 nw166 0 2f
M1029 nw167 nw90 vdd vdd pch w=2u l=180n
M1030 nw167 nw98 vdd vdd pch w=2u l=180n
CT349 t349 0 0.1f
M1031 nw167 nw90 t349 0 nch w=1u l=180n
M1032 t349 nw98 0 0 nch w=1u l=180n
Cnw167 nw167 0 2f
M1033 nw168 nw92 0 0 nch w=1u l=180n
M1034 nw168 nw101 0 0 nch w=1u l=180n
CT350 t350 0 0.1f
M1035 t350 nw92 vdd vdd pch w=2u l=180n
M1036 nw168 nw101 t350 vdd pch w=2u l=180n
Cnw168 nw168 0 2f
CT351 t351 0 0.1f
M1037 t351 nw94 vdd vdd pch w=2u l=180n
M1038 t351 nw104 vdd vdd pch w=2u l=180n
CT352 t352 0 0.1f
M1039 t351 nw94 t352 0 nch w=1u l=180n
M1040 t352 nw104 0 0 nch w=1u l=180n
M1041 nw169 t351 vdd vdd pch w=2u l=180n
M1042 nw169 t351 0 0 nch w=1u l=180n
Cnw169 nw169 0 2f
CT353 t353 0 0.1f
M1043 t353 nw96 0 0 nch w=1u l=180n
M1044 t353 nw107 0 0 nch w=1u l=180n
CT354 t354 0 0.1f
M1045 t354 nw96 vdd vdd pch w=2u l=180n
M1046 t353 nw107 t354 vdd pch w=2u l=180n
M1047 nw170 t353 vdd vdd pch w=2u l=180n
M1048 nw170 t353 0 0 nch w=1u l=180n
Cnw170 nw170 0 2f
CT355 t355 0 0.1f
CT356 t356 0 0.1f
CT357 t357 0 0.1f
M1049 t355 nw98 vdd vdd pch w=2u l=180n
M1050 t355 nw110 vdd vdd pch w=2u l=180n
CT358 t358 0 0.1f
M1051 t355 nw98 t358 0 nch w=1u l=180n
M1052 t358 nw110 0 0 nch w=1u l=180n
M1053 t356 nw98 vdd vdd pch w=2u l=180n
M1054 t356 t355 vdd vdd pch w=2u l=180n
CT359 t359 0 0.1f
M1055 t356 nw98 t359 0 nch w=1u l=180n
M1056 t359 t355 0 0 nch w=1u l=180n
M1057 t357 nw110 vdd vdd pch w=2u l=180n
M1058 t357 t355 vdd vdd pch w=2u l=180n
CT360 t360 0 0.1f
M1059 t357 nw110 t360 0 nch w=1u l=180n
M1060 t360 t355 0 0 nch w=1u l=180n
M1061 nw171 t356 vdd vdd pch w=2u l=180n
M1062 nw171 t357 vdd vdd pch w=2u l=180n
CT361 t361 0 0.1f
M1063 nw171 t356 t361 0 nch w=1u l=180n
M1064 t361 t357 0 0 nch w=1u l=180n
Cnw171 nw171 0 2f
M1065 nw172 nw100 vdd vdd pch w=2u l=180n
M1066 nw172 nw113 vdd vdd pch w=2u l=180n
CT362 t362 0 0.1f
M1067 nw172 nw100 t362 0 nch w=1u l=180n
M1068 t362 nw113 0 0 nch w=1u l=180n
Cnw172 nw172 0 2f
M1069 nw173 nw102 0 0 nch w=1u l=180n
M1070 nw173 nw116 0 0 nch w=1u l=180n
CT363 t363 0 0.1f
M1071 t363 nw102 vdd vdd pch w=2u l=180n
M1072 nw173 nw116 t363 vdd pch w=2u l=180n
Cnw173 nw173 0 2f
CT364 t364 0 0.1f
M1073 t364 nw104 vdd vdd pch w=2u l=180n
M1074 t364 nw119 vdd vdd pch w=2u l=180n
CT365 t365 0 0.1f
M1075 t364 nw104 t365 0 nch w=1u l=180n
M1076 t365 nw119 0 0 nch w=1u l=180n
M1077 nw174 t364 vdd vdd pch w=2u l=180n
M1078 nw174 t364 0 0 nch w=1u l=180n
Cnw174 nw174 0 2f
CT366 t366 0 0.1f
M1079 t366 nw106 0 0 nch w=1u l=180n
M1080 t366 nw122 0 0 nch w=1u l=180n
CT367 t367 0 0.1f
M1081 t367 nw106 vdd vdd pch w=2u l=180n
M1082 t366 nw122 t367 vdd pch w=2u l=180n
M1083 nw175 t366 vdd vdd pch w=2u l=180n
M1084 nw175 t366 0 0 nch w=1u l=180n
Cnw175 nw175 0 2f
CT368 t368 0 0.1f
CT369 t369 0 0.1f
CT370 t370 0 0.1f
M1085 t368 nw108 vdd vdd pch w=2u l=180n
M1086 t368 nw125 vdd vdd pch w=2u l=180n
CT371 t371 0 0.1f
M1087 t368 nw108 t371 0 nch w=1u l=180n
M1088 t371 nw125 0 0 nch w=1u l=180n
M1089 t369 nw108 vdd vdd pch w=2u l=180n
M1090 t369 t368 vdd vdd pch w=2u l=180n
CT372 t372 0 0.1f
M1091 t369 nw108 t372 0 nch w=1u l=180n
M1092 t372 t368 0 0 nch w=1u l=180n
M1093 t370 nw125 vdd vdd pch w=2u l=180n
M1094 t370 t368 vdd vdd pch w=2u l=180n
CT373 t373 0 0.1f
M1095 t370 nw125 t373 0 nch w=1u l=180n
M1096 t373 t368 0 0 nch w=1u l=180n
M1097 nw176 t369 vdd vdd pch w=2u l=180n
M1098 nw176 t370 vdd vdd pch w=2u l=180n
CT374 t374 0 0.1f
M1099 nw176 t369 t374 0 nch w=1u l=180n
M1100 t374 t370 0 0 nch w=1u l=180n
Cnw176 nw176 0 2f
M1101 nw177 nw110 vdd vdd pch w=2u l=180n
M1102 nw177 nw128 vdd vdd pch w=2u l=180n
CT375 t375 0 0.1f
M1103 nw177 nw110 t375 0 nch w=1u l=180n
M1104 t375 nw128 0 0 nch w=1u l=180n
Cnw177 nw177 0 2f
M1105 nw178 nw112 0 0 nch w=1u l=180n
M1106 nw178 nw131 0 0 nch w=1u l=180n
CT376 t376 0 0.1f
M1107 t376 nw112 vdd vdd pch w=2u l=180n
M1108 nw178 nw131 t376 vdd pch w=2u l=180n
Cnw178 nw178 0 2f
CT377 t377 0 0.1f
M1109 t377 nw114 vdd vdd pch w=2u l=180n
M1110 t377 nw134 vdd vdd pch w=2u l=180n
CT378 t378 0 0.1f
M1111 t377 nw114 t378 0 nch w=1u l=180n
M1112 t378 nw134 0 0 nch w=1u l=180n
M1113 nw179 t377 vdd vdd pch w=2u l=180n
M1114 nw179 t377 0 0 nch w=1u l=180n
Cnw179 nw179 0 2f
CT379 t379 0 0.1f
M1115 t379 nw116 0 0 nch w=1u l=180n
M1116 t379 nw137 0 0 nch w=1u l=180n
CT380 t380 0 0.1f
M1117 t380 nw116 vdd vdd pch w=2u l=180n
M1118 t379 nw137 t380 vdd pch w=2u l=180n
M1119 nw180 t379 vdd vdd pch w=2u l=180n
M1120 nw180 t379 0 0 nch w=1u l=180n
Cnw180 nw180 0 2f
CT381 t381 0 0.1f
CT382 t382 0 0.1f
CT383 t383 0 0.1f
M1121 t381 nw118 vdd vdd pch w=2u l=180n
M1122 t381 nw140 vdd vdd pch w=2u l=180n
CT384 t384 0 0.1f
M1123 t381 nw118 t384 0 nch w=1u l=180n
M1124 t384 nw140 0 0 nch w=1u l=180n
M1125 t382 nw118 vdd vdd pch w=2u l=180n
M1126 t382 t381 vdd vdd pch w=2u l=180n
CT385 t385 0 0.1f
M1127 t382 nw118 t385 0 nch w=1u l=180n
M1128 t385 t381 0 0 nch w=1u l=180n
M1129 t383 nw140 vdd vdd pch w=2u l=180n
M1130 t383 t381 vdd vdd pch w=2u l=180n
CT386 t386 0 0.1f
M1131 t383 nw140 t386 0 nch w=1u l=180n
M1132 t386 t381 0 0 nch w=1u l=180n
M1133 nw181 t382 vdd vdd pch w=2u l=180n
M1134 nw181 t383 vdd vdd pch w=2u l=180n
CT387 t387 0 0.1f
M1135 nw181 t382 t387 0 nch w=1u l=180n
M1136 t387 t383 0 0 nch w=1u l=180n
Cnw181 nw181 0 2f
M1137 nw182 nw120 vdd vdd pch w=2u l=180n
M1138 nw182 nw143 vdd vdd pch w=2u l=180n
CT388 t388 0 0.1f
M1139 nw182 nw120 t388 0 nch w=1u l=180n
M1140 t388 nw143 0 0 nch w=1u l=180n
Cnw182 nw182 0 2f
M1141 nw183 nw122 0 0 nch w=1u l=180n
M1142 nw183 nw146 0 0 nch w=1u l=180n
CT389 t389 0 0.1f
M1143 t389 nw122 vdd vdd pch w=2u l=180n
M1144 nw183 nw146 t389 vdd pch w=2u l=180n
Cnw183 nw183 0 2f
CT390 t390 0 0.1f
M1145 t390 nw124 vdd vdd pch w=2u l=180n
M1146 t390 nw149 vdd vdd pch w=2u l=180n
CT391 t391 0 0.1f
M1147 t390 nw124 t391 0 nch w=1u l=180n
M1148 t391 nw149 0 0 nch w=1u l=180n
M1149 nw184 t390 vdd vdd pch w=2u l=180n
M1150 nw184 t390 0 0 nch w=1u l=180n
Cnw184 nw184 0 2f
CT392 t392 0 0.1f
M1151 t392 nw126 0 0 nch w=1u l=180n
M1152 t392 nw152 0 0 nch w=1u l=180n
CT393 t393 0 0.1f
M1153 t393 nw126 vdd vdd pch w=2u l=180n
M1154 t392 nw152 t393 vdd pch w=2u l=180n
M1155 nw185 t392 vdd vdd pch w=2u l=180n
M1156 nw185 t392 0 0 nch w=1u l=180n
Cnw185 nw185 0 2f
CT394 t394 0 0.1f
CT395 t395 0 0.1f
CT396 t396 0 0.1f
M1157 t394 nw128 vdd vdd pch w=2u l=180n
M1158 t394 nw155 vdd vdd pch w=2u l=180n
CT397 t397 0 0.1f
M1159 t394 nw128 t397 0 nch w=1u l=180n
M1160 t397 nw155 0 0 nch w=1u l=180n
M1161 t395 nw128 vdd vdd pch w=2u l=180n
M1162 t395 t394 vdd vdd pch w=2u l=180n
CT398 t398 0 0.1f
M1163 t395 nw128 t398 0 nch w=1u l=180n
M1164 t398 t394 0 0 nch w=1u l=180n
M1165 t396 nw155 vdd vdd pch w=2u l=180n
M1166 t396 t394 vdd vdd pch w=2u l=180n
CT399 t399 0 0.1f
M1167 t396 nw155 t399 0 nch w=1u l=180n
M1168 t399 t394 0 0 nch w=1u l=180n
M1169 nw186 t395 vdd vdd pch w=2u l=180n
M1170 nw186 t396 vdd vdd pch w=2u l=180n
CT400 t400 0 0.1f
M1171 nw186 t395 t400 0 nch w=1u l=180n
M1172 t400 t396 0 0 nch w=1u l=180n
Cnw186 nw186 0 2f
M1173 nw187 nw130 vdd vdd pch w=2u l=180n
M1174 nw187 nw158 vdd vdd pch w=2u l=180n
CT401 t401 0 0.1f
M1175 nw187 nw130 t401 0 nch w=1u l=180n
M1176 t401 nw158 0 0 nch w=1u l=180n
Cnw187 nw187 0 2f
M1177 nw188 nw132 0 0 nch w=1u l=180n
M1178 nw188 nw161 0 0 nch w=1u l=180n
CT402 t402 0 0.1f
M1179 t402 nw132 vdd vdd pch w=2u l=180n
M1180 nw188 nw161 t402 vdd pch w=2u l=180n
Cnw188 nw188 0 2f
CT403 t403 0 0.1f
M1181 t403 nw134 vdd vdd pch w=2u l=180n
M1182 t403 nw164 vdd vdd pch w=2u l=180n
CT404 t404 0 0.1f
M1183 t403 nw134 t404 0 nch w=1u l=180n
M1184 t404 nw164 0 0 nch w=1u l=180n
M1185 nw189 t403 vdd vdd pch w=2u l=180n
M1186 nw189 t403 0 0 nch w=1u l=180n
Cnw189 nw189 0 2f
CT405 t405 0 0.1f
M1187 t405 nw136 0 0 nch w=1u l=180n
M1188 t405 nw167 0 0 nch w=1u l=180n
CT406 t406 0 0.1f
M1189 t406 nw136 vdd vdd pch w=2u l=180n
M1190 t405 nw167 t406 vdd pch w=2u l=180n
M1191 nw190 t405 vdd vdd pch w=2u l=180n
M1192 nw190 t405 0 0 nch w=1u l=180n
Cnw190 nw190 0 2f
CT407 t407 0 0.1f
CT408 t408 0 0.1f
CT409 t409 0 0.1f
M1193 t407 nw138 vdd vdd pch w=2u l=180n
M1194 t407 nw170 vdd vdd pch w=2u l=180n
CT410 t410 0 0.1f
M1195 t407 nw138 t410 0 nch w=1u l=180n
M1196 t410 nw170 0 0 nch w=1u l=180n
M1197 t408 nw138 vdd vdd pch w=2u l=180n
M1198 t408 t407 vdd vdd pch w=2u l=180n
CT411 t411 0 0.1f
M1199 t408 nw138 t411 0 nch w=1u l=180n
M1200 t411 t407 0 0 nch w=1u l=180n
M1201 t409 nw170 vdd vdd pch w=2u l=180n
M1202 t409 t407 vdd vdd pch w=2u l=180n
CT412 t412 0 0.1f
M1203 t409 nw170 t412 0 nch w=1u l=180n
M1204 t412 t407 0 0 nch w=1u l=180n
M1205 nw191 t408 vdd vdd pch w=2u l=180n
M1206 nw191 t409 vdd vdd pch w=2u l=180n
CT413 t413 0 0.1f
M1207 nw191 t408 t413 0 nch w=1u l=180n
M1208 t413 t409 0 0 nch w=1u l=180n
Cnw191 nw191 0 2f
M1209 nw192 nw140 vdd vdd pch w=2u l=180n
M1210 nw192 nw173 vdd vdd pch w=2u l=180n
CT414 t414 0 0.1f
M1211 nw192 nw140 t414 0 nch w=1u l=180n
M1212 t414 nw173 0 0 nch w=1u l=180n
Cnw192 nw192 0 2f
M1213 nw193 nw142 0 0 nch w=1u l=180n
M1214 nw193 nw176 0 0 nch w=1u l=180n
CT415 t415 0 0.1f
M1215 t415 nw142 vdd vdd pch w=2u l=180n
M1216 nw193 nw176 t415 vdd pch w=2u l=180n
Cnw193 nw193 0 2f
CT416 t416 0 0.1f
M1217 t416 nw144 vdd vdd pch w=2u l=180n
M1218 t416 nw179 vdd vdd pch w=2u l=180n
CT417 t417 0 0.1f
M1219 t416 nw144 t417 0 nch w=1u l=180n
M1220 t417 nw179 0 0 nch w=1u l=180n
M1221 nw194 t416 vdd vdd pch w=2u l=180n
M1222 nw194 t416 0 0 nch w=1u l=180n
Cnw194 nw194 0 2f
CT418 t418 0 0.1f
M1223 t418 nw146 0 0 nch w=1u l=180n
M1224 t418 nw182 0 0 nch w=1u l=180n
CT419 t419 0 0.1f
M1225 t419 nw146 vdd vdd pch w=2u l=180n
M1226 t418 nw182 t419 vdd pch w=2u l=180n
M1227 nw195 t418 vdd vdd pch w=2u l=180n
M1228 nw195 t418 0 0 nch w=1u l=180n
Cnw195 nw195 0 2f
CT420 t420 0 0.1f
CT421 t421 0 0.1f
CT422 t422 0 0.1f
M1229 t420 nw148 vdd vdd pch w=2u l=180n
M1230 t420 nw185 vdd vdd pch w=2u l=180n
CT423 t423 0 0.1f
M1231 t420 nw148 t423 0 nch w=1u l=180n
M1232 t423 nw185 0 0 nch w=1u l=180n
M1233 t421 nw148 vdd vdd pch w=2u l=180n
M1234 t421 t420 vdd vdd pch w=2u l=180n
CT424 t424 0 0.1f
M1235 t421 nw148 t424 0 nch w=1u l=180n
M1236 t424 t420 0 0 nch w=1u l=180n
M1237 t422 nw185 vdd vdd pch w=2u l=180n
M1238 t422 t420 vdd vdd pch w=2u l=180n
CT425 t425 0 0.1f
M1239 t422 nw185 t425 0 nch w=1u l=180n
M1240 t425 t420 0 0 nch w=1u l=180n
M1241 nw196 t421 vdd vdd pch w=2u l=180n
M1242 nw196 t422 vdd vdd pch w=2u l=180n
CT426 t426 0 0.1f
M1243 nw196 t421 t426 0 nch w=1u l=180n
M1244 t426 t422 0 0 nch w=1u l=180n
Cnw196 nw196 0 2f
M1245 nw197 nw150 vdd vdd pch w=2u l=180n
M1246 nw197 nw188 vdd vdd pch w=2u l=180n
CT427 t427 0 0.1f
M1247 nw197 nw150 t427 0 nch w=1u l=180n
M1248 t427 nw188 0 0 nch w=1u l=180n
Cnw197 nw197 0 2f
M1249 nw198 nw152 0 0 nch w=1u l=180n
M1250 nw198 nw191 0 0 nch w=1u l=180n
CT428 t428 0 0.1f
M1251 t428 nw152 vdd vdd pch w=2u l=180n
M1252 nw198 nw191 t428 vdd pch w=2u l=180n
Cnw198 nw198 0 2f
CT429 t429 0 0.1f
M1253 t429 nw154 vdd vdd pch w=2u l=180n
M1254 t429 nw194 vdd vdd pch w=2u l=180n
CT430 t430 0 0.1f
M1255 t429 nw154 t430 0 nch w=1u l=180n
M1256 t430 nw194 0 0 nch w=1u l=180n
M1257 nw199 t429 vdd vdd pch w=2u l=180n
M1258 nw199 t429 0 0 nch w=1u l=180n
Cnw199 nw199 0 2f
CT431 t431 0 0.1f
M1259 t431 nw156 0 0 nch w=1u l=180n
M1260 t431 nw197 0 0 nch w=1u l=180n
CT432 t432 0 0.1f
M1261 t432 nw156 vdd vdd pch w=2u l=180n
M1262 t431 nw197 t432 vdd pch w=2u l=180n
M1263 nw200 t431 vdd vdd pch w=2u l=180n
M1264 nw200 t431 0 0 nch w=1u l=180n
Cnw200 nw200 0 2f
CT433 t433 0 0.1f
CT434 t434 0 0.1f
CT435 t435 0 0.1f
M1265 t433 nw158 vdd vdd pch w=2u l=180n
M1266 t433 nw200 vdd vdd pch w=2u l=180n
CT436 t436 0 0.1f
M1267 t433 nw158 t436 0 nch w=1u l=180n
M1268 t436 nw200 0 0 nch w=1u l=180n
M1269 t434 nw158 vdd vdd pch w=2u l=180n
M1270 t434 t433 vdd vdd pch w=2u l=180n
CT437 t437 0 0.1f
M1271 t434 nw158 t437 0 nch w=1u l=180n
M1272 t437 t433 0 0 nch w=1u l=180n
M1273 t435 nw200 vdd vdd pch w=2u l=180n
M1274 t435 t433 vdd vdd pch w=2u l=180n
CT438 t438 0 0.1f
M1275 t435 nw200 t438 0 nch w=1u l=180n
M1276 t438 t433 0 0 nch w=1u l=180n
M1277 nw201 t434 vdd vdd pch w=2u l=180n
M1278 nw201 t435 vdd vdd pch w=2u l=180n
CT439 t439 0 0.1f
M1279 nw201 t434 t439 0 nch w=1u l=180n
M1280 t439 t435 0 0 nch w=1u l=180n
Cnw201 nw201 0 2f
M1281 nw202 nw160 vdd vdd pch w=2u l=180n
M1282 nw202 nq1 vdd vdd pch w=2u l=180n
CT440 t440 0 0.1f
M1283 nw202 nw160 t440 0 nch w=1u l=180n
M1284 t440 nq1 0 0 nch w=1u l=180n
Cnw202 nw202 0 2f
M1285 nw203 nw162 0 0 nch w=1u l=180n
M1286 nw203 nq3 0 0 nch w=1u l=180n
CT441 t441 0 0.1f
M1287 t441 nw162 vdd vdd pch w=2u l=180n
M1288 nw203 nq3 t441 vdd pch w=2u l=180n
Cnw203 nw203 0 2f
CT442 t442 0 0.1f
M1289 t442 nw164 vdd vdd pch w=2u l=180n
M1290 t442 nq5 vdd vdd pch w=2u l=180n
CT443 t443 0 0.1f
M1291 t442 nw164 t443 0 nch w=1u l=180n
M1292 t443 nq5 0 0 nch w=1u l=180n
M1293 nw204 t442 vdd vdd pch w=2u l=180n
M1294 nw204 t442 0 0 nch w=1u l=180n
Cnw204 nw204 0 2f
CT444 t444 0 0.1f
M1295 t444 nw166 0 0 nch w=1u l=180n
M1296 t444 nq7 0 0 nch w=1u l=180n
CT445 t445 0 0.1f
M1297 t445 nw166 vdd vdd pch w=2u l=180n
M1298 t444 nq7 t445 vdd pch w=2u l=180n
M1299 nw205 t444 vdd vdd pch w=2u l=180n
M1300 nw205 t444 0 0 nch w=1u l=180n
Cnw205 nw205 0 2f
CT446 t446 0 0.1f
CT447 t447 0 0.1f
CT448 t448 0 0.1f
M1301 t446 nw168 vdd vdd pch w=2u l=180n
M1302 t446 nq9 vdd vdd pch w=2u l=180n
CT449 t449 0 0.1f
M1303 t446 nw168 t449 0 nch w=1u l=180n
M1304 t449 nq9 0 0 nch w=1u l=180n
M1305 t447 nw168 vdd vdd pch w=2u l=180n
M1306 t447 t446 vdd vdd pch w=2u l=180n
CT450 t450 0 0.1f
M1307 t447 nw168 t450 0 nch w=1u l=180n
M1308 t450 t446 0 0 nch w=1u l=180n
M1309 t448 nq9 vdd vdd pch w=2u l=180n
M1310 t448 t446 vdd vdd pch w=2u l=180n
CT451 t451 0 0.1f
M1311 t448 nq9 t451 0 nch w=1u l=180n
M1312 t451 t446 0 0 nch w=1u l=180n
M1313 nw206 t447 vdd vdd pch w=2u l=180n
M1314 nw206 t448 vdd vdd pch w=2u l=180n
CT452 t452 0 0.1f
M1315 nw206 t447 t452 0 nch w=1u l=180n
M1316 t452 t448 0 0 nch w=1u l=180n
Cnw206 nw206 0 2f
M1317 nw207 nw170 vdd vdd pch w=2u l=180n
M1318 nw207 nq11 vdd vdd pch w=2u l=180n
CT453 t453 0 0.1f
M1319 nw207 nw170 t453 0 nch w=1u l=180n
M1320 t453 nq11 0 0 nch w=1u l=180n
Cnw207 nw207 0 2f
M1321 nw208 nw172 0 0 nch w=1u l=180n
M1322 nw208 nq13 0 0 nch w=1u l=180n
CT454 t454 0 0.1f
M1323 t454 nw172 vdd vdd pch w=2u l=180n
M1324 nw208 nq13 t454 vdd pch w=2u l=180n
Cnw208 nw208 0 2f
CT455 t455 0 0.1f
M1325 t455 nw174 vdd vdd pch w=2u l=180n
M1326 t455 nq15 vdd vdd pch w=2u l=180n
CT456 t456 0 0.1f
M1327 t455 nw174 t456 0 nch w=1u l=180n
M1328 t456 nq15 0 0 nch w=1u l=180n
M1329 nw209 t455 vdd vdd pch w=2u l=180n
M1330 nw209 t455 0 0 nch w=1u l=180n
Cnw209 nw209 0 2f
CT457 t457 0 0.1f
M1331 t457 nw176 0 0 nch w=1u l=180n
M1332 t457 nq17 0 0 nch w=1u l=180n
CT458 t458 0 0.1f
M1333 t458 nw176 vdd vdd pch w=2u l=180n
M1334 t457 nq17 t458 vdd pch w=2u l=180n
M1335 nw210 t457 vdd vdd pch w=2u l=180n
M1336 nw210 t457 0 0 nch w=1u l=180n
Cnw210 nw210 0 2f
CT459 t459 0 0.1f
CT460 t460 0 0.1f
CT461 t461 0 0.1f
M1337 t459 nw178 vdd vdd pch w=2u l=180n
M1338 t459 ni0 vdd vdd pch w=2u l=180n
CT462 t462 0 0.1f
M1339 t459 nw178 t462 0 nch w=1u l=180n
M1340 t462 ni0 0 0 nch w=1u l=180n
M1341 t460 nw178 vdd vdd pch w=2u l=180n
M1342 t460 t459 vdd vdd pch w=2u l=180n
CT463 t463 0 0.1f
M1343 t460 nw178 t463 0 nch w=1u l=180n
M1344 t463 t459 0 0 nch w=1u l=180n
M1345 t461 ni0 vdd vdd pch w=2u l=180n
M1346 t461 t459 vdd vdd pch w=2u l=180n
CT464 t464 0 0.1f
M1347 t461 ni0 t464 0 nch w=1u l=180n
M1348 t464 t459 0 0 nch w=1u l=180n
M1349 nw211 t460 vdd vdd pch w=2u l=180n
M1350 nw211 t461 vdd vdd pch w=2u l=180n
CT465 t465 0 0.1f
M1351 nw211 t460 t465 0 nch w=1u l=180n
M1352 t465 t461 0 0 nch w=1u l=180n
Cnw211 nw211 0 2f
M1353 nw212 nw180 vdd vdd pch w=2u l=180n
M1354 nw212 ni2 vdd vdd pch w=2u l=180n
CT466 t466 0 0.1f
M1355 nw212 nw180 t466 0 nch w=1u l=180n
M1356 t466 ni2 0 0 nch w=1u l=180n
Cnw212 nw212 0 2f
M1357 nw213 nw182 0 0 nch w=1u l=180n
M1358 nw213 ni4 0 0 nch w=1u l=180n
CT467 t467 0 0.1f
M1359 t467 nw182 vdd vdd pch w=2u l=180n
M1360 nw213 ni4 t467 vdd pch w=2u l=180n
Cnw213 nw213 0 2f
CT468 t468 0 0.1f
M1361 t468 nw184 vdd vdd pch w=2u l=180n
M1362 t468 ni6 vdd vdd pch w=2u l=180n
CT469 t469 0 0.1f
M1363 t468 nw184 t469 0 nch w=1u l=180n
M1364 t469 ni6 0 0 nch w=1u l=180n
M1365 nw214 t468 vdd vdd pch w=2u l=180n
M1366 nw214 t468 0 0 nch w=1u l=180n
Cnw214 nw214 0 2f
CT470 t470 0 0.1f
M1367 t470 nw186 0 0 nch w=1u l=180n
M1368 t470 ni8 0 0 nch w=1u l=180n
CT471 t471 0 0.1f
M1369 t471 nw186 vdd vdd pch w=2u l=180n
M1370 t470 ni8 t471 vdd pch w=2u l=180n
M1371 nw215 t470 vdd vdd pch w=2u l=180n
M1372 nw215 t470 0 0 nch w=1u l=180n
Cnw215 nw215 0 2f
CT472 t472 0 0.1f
CT473 t473 0 0.1f
CT474 t474 0 0.1f
M1373 t472 nw188 vdd vdd pch w=2u l=180n
M1374 t472 nw78 vdd vdd pch w=2u l=180n
CT475 t475 0 0.1f
M1375 t472 nw188 t475 0 nch w=1u l=180n
M1376 t475 nw78 0 0 nch w=1u l=180n
M1377 t473 nw188 vdd vdd pch w=2u l=180n
M1378 t473 t472 vdd vdd pch w=2u l=180n
CT476 t476 0 0.1f
M1379 t473 nw188 t476 0 nch w=1u l=180n
M1380 t476 t472 0 0 nch w=1u l=180n
M1381 t474 nw78 vdd vdd pch w=2u l=180n
M1382 t474 t472 vdd vdd pch w=2u l=180n
CT477 t477 0 0.1f
M1383 t474 nw78 t477 0 nch w=1u l=180n
M1384 t477 t472 0 0 nch w=1u l=180n
M1385 nw216 t473 vdd vdd pch w=2u l=180n
M1386 nw216 t474 vdd vdd pch w=2u l=180n
CT478 t478 0 0.1f
M1387 nw216 t473 t478 0 nch w=1u l=180n
M1388 t478 t474 0 0 nch w=1u l=180n
Cnw216 nw216 0 2f
M1389 nw217 nw190 vdd vdd pch w=2u l=180n
M1390 nw217 nw80 vdd vdd pch w=2u l=180n
CT479 t479 0 0.1f
M1391 nw217 nw190 t479 0 nch w=1u l=180n
M1392 t479 nw80 0 0 nch w=1u l=180n
Cnw217 nw217 0 2f
M1393 nw218 nw192 0 0 nch w=1u l=180n
M1394 nw218 nw82 0 0 nch w=1u l=180n
CT480 t480 0 0.1f
M1395 t480 nw192 vdd vdd pch w=2u l=180n
M1396 nw218 nw82 t480 vdd pch w=2u l=180n
Cnw218 nw218 0 2f
CT481 t481 0 0.1f
M1397 t481 nw194 vdd vdd pch w=2u l=180n
M1398 t481 nw84 vdd vdd pch w=2u l=180n
CT482 t482 0 0.1f
M1399 t481 nw194 t482 0 nch w=1u l=180n
M1400 t482 nw84 0 0 nch w=1u l=180n
M1401 nw219 t481 vdd vdd pch w=2u l=180n
M1402 nw219 t481 0 0 nch w=1u l=180n
Cnw219 nw219 0 2f
CT483 t483 0 0.1f
M1403 t483 nw196 0 0 nch w=1u l=180n
M1404 t483 nw86 0 0 nch w=1u l=180n
CT484 t484 0 0.1f
M1405 t484 nw196 vdd vdd pch w=2u l=180n
M1406 t483 nw86 t484 vdd pch w=2u l=180n
M1407 nw220 t483 vdd vdd pch w=2u l=180n
M1408 nw220 t483 0 0 nch w=1u l=180n
Cnw220 nw220 0 2f
CT485 t485 0 0.1f
CT486 t486 0 0.1f
CT487 t487 0 0.1f
M1409 t485 nw198 vdd vdd pch w=2u l=180n
M1410 t485 nw88 vdd vdd pch w=2u l=180n
CT488 t488 0 0.1f
M1411 t485 nw198 t488 0 nch w=1u l=180n
M1412 t488 nw88 0 0 nch w=1u l=180n
M1413 t486 nw198 vdd vdd pch w=2u l=180n
M1414 t486 t485 vdd vdd pch w=2u l=180n
CT489 t489 0 0.1f
M1415 t486 nw198 t489 0 nch w=1u l=180n
M1416 t489 t485 0 0 nch w=1u l=180n
M1417 t487 nw88 vdd vdd pch w=2u l=180n
M1418 t487 t485 vdd vdd pch w=2u l=180n
CT490 t490 0 0.1f
M1419 t487 nw88 t490 0 nch w=1u l=180n
M1420 t490 t485 0 0 nch w=1u l=180n
M1421 nw221 t486 vdd vdd pch w=2u l=180n
M1422 nw221 t487 vdd vdd pch w=2u l=180n
CT491 t491 0 0.1f
M1423 nw221 t486 t491 0 nch w=1u l=180n
M1424 t491 t487 0 0 nch w=1u l=180n
Cnw221 nw221 0 2f
M1425 nw222 nw200 vdd vdd pch w=2u l=180n
M1426 nw222 nw90 vdd vdd pch w=2u l=180n
CT492 t492 0 0.1f
M1427 nw222 nw200 t492 0 nch w=1u l=180n
M1428 t492 nw90 0 0 nch w=1u l=180n
Cnw222 nw222 0 2f
M1429 nw223 nw202 0 0 nch w=1u l=180n
M1430 nw223 nw92 0 0 nch w=1u l=180n
CT493 t493 0 0.1f
M1431 t493 nw202 vdd vdd pch w=2u l=180n
M1432 nw223 nw92 t493 vdd pch w=2u l=180n
Cnw223 nw223 0 2f
CT494 t494 0 0.1f
M1433 t494 nw204 vdd vdd pch w=2u l=180n
M1434 t494 nw94 vdd vdd pch w=2u l=180n
CT495 t495 0 0.1f
M1435 t494 nw204 t495 0 nch w=1u l=180n
M1436 t495 nw94 0 0 nch w=1u l=180n
M1437 nw224 t494 vdd vdd pch w=2u l=180n
M1438 nw224 t494 0 0 nch w=1u l=180n
Cnw224 nw224 0 2f
CT496 t496 0 0.1f
M1439 t496 nw206 0 0 nch w=1u l=180n
M1440 t496 nw96 0 0 nch w=1u l=180n
CT497 t497 0 0.1f
M1441 t497 nw206 vdd vdd pch w=2u l=180n
M1442 t496 nw96 t497 vdd pch w=2u l=180n
M1443 nw225 t496 vdd vdd pch w=2u l=180n
M1444 nw225 t496 0 0 nch w=1u l=180n
Cnw225 nw225 0 2f
CT498 t498 0 0.1f
CT499 t499 0 0.1f
CT500 t500 0 0.1f
M1445 t498 nw208 vdd vdd pch w=2u l=180n
M1446 t498 nw98 vdd vdd pch w=2u l=180n
CT501 t501 0 0.1f
M1447 t498 nw208 t501 0 nch w=1u l=180n
M1448 t501 nw98 0 0 nch w=1u l=180n
M1449 t499 nw208 vdd vdd pch w=2u l=180n
M1450 t499 t498 vdd vdd pch w=2u l=180n
CT502 t502 0 0.1f
M1451 t499 nw208 t502 0 nch w=1u l=180n
M1452 t502 t498 0 0 nch w=1u l=180n
M1453 t500 nw98 vdd vdd pch w=2u l=180n
M1454 t500 t498 vdd vdd pch w=2u l=180n
CT503 t503 0 0.1f
M1455 t500 nw98 t503 0 nch w=1u l=180n
M1456 t503 t498 0 0 nch w=1u l=180n
M1457 nw226 t499 vdd vdd pch w=2u l=180n
M1458 nw226 t500 vdd vdd pch w=2u l=180n
CT504 t504 0 0.1f
M1459 nw226 t499 t504 0 nch w=1u l=180n
M1460 t504 t500 0 0 nch w=1u l=180n
Cnw226 nw226 0 2f
M1461 nw227 nw210 vdd vdd pch w=2u l=180n
M1462 nw227 nw100 vdd vdd pch w=2u l=180n
CT505 t505 0 0.1f
M1463 nw227 nw210 t505 0 nch w=1u l=180n
M1464 t505 nw100 0 0 nch w=1u l=180n
Cnw227 nw227 0 2f
M1465 nw228 nw212 0 0 nch w=1u l=180n
M1466 nw228 nw102 0 0 nch w=1u l=180n
CT506 t506 0 0.1f
M1467 t506 nw212 vdd vdd pch w=2u l=180n
M1468 nw228 nw102 t506 vdd pch w=2u l=180n
Cnw228 nw228 0 2f
CT507 t507 0 0.1f
M1469 t507 nw214 vdd vdd pch w=2u l=180n
M1470 t507 nw104 vdd vdd pch w=2u l=180n
CT508 t508 0 0.1f
M1471 t507 nw214 t508 0 nch w=1u l=180n
M1472 t508 nw104 0 0 nch w=1u l=180n
M1473 nw229 t507 vdd vdd pch w=2u l=180n
M1474 nw229 t507 0 0 nch w=1u l=180n
Cnw229 nw229 0 2f
CT509 t509 0 0.1f
M1475 t509 nw216 0 0 nch w=1u l=180n
M1476 t509 nw106 0 0 nch w=1u l=180n
CT510 t510 0 0.1f
M1477 t510 nw216 vdd vdd pch w=2u l=180n
M1478 t509 nw106 t510 vdd pch w=2u l=180n
M1479 nw230 t509 vdd vdd pch w=2u l=180n
M1480 nw230 t509 0 0 nch w=1u l=180n
Cnw230 nw230 0 2f
CT511 t511 0 0.1f
CT512 t512 0 0.1f
CT513 t513 0 0.1f
M1481 t511 nw218 vdd vdd pch w=2u l=180n
M1482 t511 nw108 vdd vdd pch w=2u l=180n
CT514 t514 0 0.1f
M1483 t511 nw218 t514 0 nch w=1u l=180n
M1484 t514 nw108 0 0 nch w=1u l=180n
M1485 t512 nw218 vdd vdd pch w=2u l=180n
M1486 t512 t511 vdd vdd pch w=2u l=180n
CT515 t515 0 0.1f
M1487 t512 nw218 t515 0 nch w=1u l=180n
M1488 t515 t511 0 0 nch w=1u l=180n
M1489 t513 nw108 vdd vdd pch w=2u l=180n
M1490 t513 t511 vdd vdd pch w=2u l=180n
CT516 t516 0 0.1f
M1491 t513 nw108 t516 0 nch w=1u l=180n
M1492 t516 t511 0 0 nch w=1u l=180n
M1493 nw231 t512 vdd vdd pch w=2u l=180n
M1494 nw231 t513 vdd vdd pch w=2u l=180n
CT517 t517 0 0.1f
M1495 nw231 t512 t517 0 nch w=1u l=180n
M1496 t517 t513 0 0 nch w=1u l=180n
Cnw231 nw231 0 2f
M1497 nw232 nw220 vdd vdd pch w=2u l=180n
M1498 nw232 nw110 vdd vdd pch w=2u l=180n
CT518 t518 0 0.1f
M1499 nw232 nw220 t518 0 nch w=1u l=180n
M1500 t518 nw110 0 0 nch w=1u l=180n
Cnw232 nw232 0 2f
M1501 nw233 nw222 0 0 nch w=1u l=180n
M1502 nw233 nw112 0 0 nch w=1u l=180n
CT519 t519 0 0.1f
M1503 t519 nw222 vdd vdd pch w=2u l=180n
M1504 nw233 nw112 t519 vdd pch w=2u l=180n
Cnw233 nw233 0 2f
CT520 t520 0 0.1f
M1505 t520 nw224 vdd vdd pch w=2u l=180n
M1506 t520 nw114 vdd vdd pch w=2u l=180n
CT521 t521 0 0.1f
M1507 t520 nw224 t521 0 nch w=1u l=180n
M1508 t521 nw114 0 0 nch w=1u l=180n
M1509 nw234 t520 vdd vdd pch w=2u l=180n
M1510 nw234 t520 0 0 nch w=1u l=180n
Cnw234 nw234 0 2f
CT522 t522 0 0.1f
M1511 t522 nw226 0 0 nch w=1u l=180n
M1512 t522 nw116 0 0 nch w=1u l=180n
CT523 t523 0 0.1f
M1513 t523 nw226 vdd vdd pch w=2u l=180n
M1514 t522 nw116 t523 vdd pch w=2u l=180n
M1515 nw235 t522 vdd vdd pch w=2u l=180n
M1516 nw235 t522 0 0 nch w=1u l=180n
Cnw235 nw235 0 2f
CT524 t524 0 0.1f
CT525 t525 0 0.1f
CT526 t526 0 0.1f
M1517 t524 nw228 vdd vdd pch w=2u l=180n
M1518 t524 nw118 vdd vdd pch w=2u l=180n
CT527 t527 0 0.1f
M1519 t524 nw228 t527 0 nch w=1u l=180n
M1520 t527 nw118 0 0 nch w=1u l=180n
M1521 t525 nw228 vdd vdd pch w=2u l=180n
M1522 t525 t524 vdd vdd pch w=2u l=180n
CT528 t528 0 0.1f
M1523 t525 nw228 t528 0 nch w=1u l=180n
M1524 t528 t524 0 0 nch w=1u l=180n
M1525 t526 nw118 vdd vdd pch w=2u l=180n
M1526 t526 t524 vdd vdd pch w=2u l=180n
CT529 t529 0 0.1f
M1527 t526 nw118 t529 0 nch w=1u l=180n
M1528 t529 t524 0 0 nch w=1u l=180n
M1529 nw236 t525 vdd vdd pch w=2u l=180n
M1530 nw236 t526 vdd vdd pch w=2u l=180n
CT530 t530 0 0.1f
M1531 nw236 t525 t530 0 nch w=1u l=180n
M1532 t530 t526 0 0 nch w=1u l=180n
Cnw236 nw236 0 2f
M1533 nw237 nw230 vdd vdd pch w=2u l=180n
M1534 nw237 nw120 vdd vdd pch w=2u l=180n
CT531 t531 0 0.1f
M1535 nw237 nw230 t531 0 nch w=1u l=180n
M1536 t531 nw120 0 0 nch w=1u l=180n
Cnw237 nw237 0 2f
M1537 nw238 nw232 0 0 nch w=1u l=180n
M1538 nw238 nw122 0 0 nch w=1u l=180n
CT532 t532 0 0.1f
M1539 t532 nw232 vdd vdd pch w=2u l=180n
M1540 nw238 nw122 t532 vdd pch w=2u l=180n
Cnw238 nw238 0 2f
CT533 t533 0 0.1f
M1541 t533 nw234 vdd vdd pch w=2u l=180n
M1542 t533 nw124 vdd vdd pch w=2u l=180n
CT534 t534 0 0.1f
M1543 t533 nw234 t534 0 nch w=1u l=180n
M1544 t534 nw124 0 0 nch w=1u l=180n
M1545 nw239 t533 vdd vdd pch w=2u l=180n
M1546 nw239 t533 0 0 nch w=1u l=180n
Cnw239 nw239 0 2f
CT535 t535 0 0.1f
M1547 t535 nw236 0 0 nch w=1u l=180n
M1548 t535 nw126 0 0 nch w=1u l=180n
CT536 t536 0 0.1f
M1549 t536 nw236 vdd vdd pch w=2u l=180n
M1550 t535 nw126 t536 vdd pch w=2u l=180n
M1551 nw240 t535 vdd vdd pch w=2u l=180n
M1552 nw240 t535 0 0 nch w=1u l=180n
Cnw240 nw240 0 2f
CT537 t537 0 0.1f
CT538 t538 0 0.1f
CT539 t539 0 0.1f
M1553 t537 nw238 vdd vdd pch w=2u l=180n
M1554 t537 nw128 vdd vdd pch w=2u l=180n
CT540 t540 0 0.1f
M1555 t537 nw238 t540 0 nch w=1u l=180n
M1556 t540 nw128 0 0 nch w=1u l=180n
M1557 t538 nw238 vdd vdd pch w=2u l=180n
M1558 t538 t537 vdd vdd pch w=2u l=180n
CT541 t541 0 0.1f
M1559 t538 nw238 t541 0 nch w=1u l=180n
M1560 t541 t537 0 0 nch w=1u l=180n
M1561 t539 nw128 vdd vdd pch w=2u l=180n
M1562 t539 t537 vdd vdd pch w=2u l=180n
CT542 t542 0 0.1f
M1563 t539 nw128 t542 0 nch w=1u l=180n
M1564 t542 t537 0 0 nch w=1u l=180n
M1565 nw241 t538 vdd vdd pch w=2u l=180n
M1566 nw241 t539 vdd vdd pch w=2u l=180n
CT543 t543 0 0.1f
M1567 nw241 t538 t543 0 nch w=1u l=180n
M1568 t543 t539 0 0 nch w=1u l=180n
Cnw241 nw241 0 2f
M1569 nw242 nw240 vdd vdd pch w=2u l=180n
M1570 nw242 nw130 vdd vdd pch w=2u l=180n
CT544 t544 0 0.1f
M1571 nw242 nw240 t544 0 nch w=1u l=180n
M1572 t544 nw130 0 0 nch w=1u l=180n
Cnw242 nw242 0 2f
M1573 nw243 nw242 0 0 nch w=1u l=180n
M1574 nw243 nw132 0 0 nch w=1u l=180n
CT545 t545 0 0.1f
M1575 t545 nw242 vdd vdd pch w=2u l=180n
M1576 nw243 nw132 t545 vdd pch w=2u l=180n
Cnw243 nw243 0 2f
CT546 t546 0 0.1f
M1577 t546 nq0 vdd vdd pch w=2u l=180n
M1578 t546 nw134 vdd vdd pch w=2u l=180n
CT547 t547 0 0.1f
M1579 t546 nq0 t547 0 nch w=1u l=180n
M1580 t547 nw134 0 0 nch w=1u l=180n
M1581 nw244 t546 vdd vdd pch w=2u l=180n
M1582 nw244 t546 0 0 nch w=1u l=180n
Cnw244 nw244 0 2f
CT548 t548 0 0.1f
M1583 t548 nq1 0 0 nch w=1u l=180n
M1584 t548 nw136 0 0 nch w=1u l=180n
CT549 t549 0 0.1f
M1585 t549 nq1 vdd vdd pch w=2u l=180n
M1586 t548 nw136 t549 vdd pch w=2u l=180n
M1587 nw245 t548 vdd vdd pch w=2u l=180n
M1588 nw245 t548 0 0 nch w=1u l=180n
Cnw245 nw245 0 2f
CT550 t550 0 0.1f
CT551 t551 0 0.1f
CT552 t552 0 0.1f
M1589 t550 nq2 vdd vdd pch w=2u l=180n
M1590 t550 nw138 vdd vdd pch w=2u l=180n
CT553 t553 0 0.1f
M1591 t550 nq2 t553 0 nch w=1u l=180n
M1592 t553 nw138 0 0 nch w=1u l=180n
M1593 t551 nq2 vdd vdd pch w=2u l=180n
M1594 t551 t550 vdd vdd pch w=2u l=180n
CT554 t554 0 0.1f
M1595 t551 nq2 t554 0 nch w=1u l=180n
M1596 t554 t550 0 0 nch w=1u l=180n
M1597 t552 nw138 vdd vdd pch w=2u l=180n
M1598 t552 t550 vdd vdd pch w=2u l=180n
CT555 t555 0 0.1f
M1599 t552 nw138 t555 0 nch w=1u l=180n
M1600 t555 t550 0 0 nch w=1u l=180n
M1601 nw246 t551 vdd vdd pch w=2u l=180n
M1602 nw246 t552 vdd vdd pch w=2u l=180n
CT556 t556 0 0.1f
M1603 nw246 t551 t556 0 nch w=1u l=180n
M1604 t556 t552 0 0 nch w=1u l=180n
Cnw246 nw246 0 2f
M1605 nw247 nq3 vdd vdd pch w=2u l=180n
M1606 nw247 nw140 vdd vdd pch w=2u l=180n
CT557 t557 0 0.1f
M1607 nw247 nq3 t557 0 nch w=1u l=180n
M1608 t557 nw140 0 0 nch w=1u l=180n
Cnw247 nw247 0 2f
M1609 nw248 nq4 0 0 nch w=1u l=180n
M1610 nw248 nw142 0 0 nch w=1u l=180n
CT558 t558 0 0.1f
M1611 t558 nq4 vdd vdd pch w=2u l=180n
M1612 nw248 nw142 t558 vdd pch w=2u l=180n
Cnw248 nw248 0 2f
CT559 t559 0 0.1f
M1613 t559 nq5 vdd vdd pch w=2u l=180n
M1614 t559 nw144 vdd vdd pch w=2u l=180n
CT560 t560 0 0.1f
M1615 t559 nq5 t560 0 nch w=1u l=180n
M1616 t560 nw144 0 0 nch w=1u l=180n
M1617 nw249 t559 vdd vdd pch w=2u l=180n
M1618 nw249 t559 0 0 nch w=1u l=180n
Cnw249 nw249 0 2f
CT561 t561 0 0.1f
M1619 t561 nq6 0 0 nch w=1u l=180n
M1620 t561 nw146 0 0 nch w=1u l=180n
CT562 t562 0 0.1f
M1621 t562 nq6 vdd vdd pch w=2u l=180n
M1622 t561 nw146 t562 vdd pch w=2u l=180n
M1623 nw250 t561 vdd vdd pch w=2u l=180n
M1624 nw250 t561 0 0 nch w=1u l=180n
Cnw250 nw250 0 2f
CT563 t563 0 0.1f
CT564 t564 0 0.1f
CT565 t565 0 0.1f
M1625 t563 nq7 vdd vdd pch w=2u l=180n
M1626 t563 nw148 vdd vdd pch w=2u l=180n
CT566 t566 0 0.1f
M1627 t563 nq7 t566 0 nch w=1u l=180n
M1628 t566 nw148 0 0 nch w=1u l=180n
M1629 t564 nq7 vdd vdd pch w=2u l=180n
M1630 t564 t563 vdd vdd pch w=2u l=180n
CT567 t567 0 0.1f
M1631 t564 nq7 t567 0 nch w=1u l=180n
M1632 t567 t563 0 0 nch w=1u l=180n
M1633 t565 nw148 vdd vdd pch w=2u l=180n
M1634 t565 t563 vdd vdd pch w=2u l=180n
CT568 t568 0 0.1f
M1635 t565 nw148 t568 0 nch w=1u l=180n
M1636 t568 t563 0 0 nch w=1u l=180n
M1637 nw251 t564 vdd vdd pch w=2u l=180n
M1638 nw251 t565 vdd vdd pch w=2u l=180n
CT569 t569 0 0.1f
M1639 nw251 t564 t569 0 nch w=1u l=180n
M1640 t569 t565 0 0 nch w=1u l=180n
Cnw251 nw251 0 2f
M1641 nw252 nq8 vdd vdd pch w=2u l=180n
M1642 nw252 nw150 vdd vdd pch w=2u l=180n
CT570 t570 0 0.1f
M1643 nw252 nq8 t570 0 nch w=1u l=180n
M1644 t570 nw150 0 0 nch w=1u l=180n
Cnw252 nw252 0 2f
M1645 nw253 nq9 0 0 nch w=1u l=180n
M1646 nw253 nw152 0 0 nch w=1u l=180n
CT571 t571 0 0.1f
M1647 t571 nq9 vdd vdd pch w=2u l=180n
M1648 nw253 nw152 t571 vdd pch w=2u l=180n
Cnw253 nw253 0 2f
CT572 t572 0 0.1f
M1649 t572 nq10 vdd vdd pch w=2u l=180n
M1650 t572 nw154 vdd vdd pch w=2u l=180n
CT573 t573 0 0.1f
M1651 t572 nq10 t573 0 nch w=1u l=180n
M1652 t573 nw154 0 0 nch w=1u l=180n
M1653 nw254 t572 vdd vdd pch w=2u l=180n
M1654 nw254 t572 0 0 nch w=1u l=180n
Cnw254 nw254 0 2f
CT574 t574 0 0.1f
M1655 t574 nq11 0 0 nch w=1u l=180n
M1656 t574 nw156 0 0 nch w=1u l=180n
CT575 t575 0 0.1f
M1657 t575 nq11 vdd vdd pch w=2u l=180n
M1658 t574 nw156 t575 vdd pch w=2u l=180n
M1659 nw255 t574 vdd vdd pch w=2u l=180n
M1660 nw255 t574 0 0 nch w=1u l=180n
Cnw255 nw255 0 2f
CT576 t576 0 0.1f
CT577 t577 0 0.1f
CT578 t578 0 0.1f
M1661 t576 nq12 vdd vdd pch w=2u l=180n
M1662 t576 nw158 vdd vdd pch w=2u l=180n
CT579 t579 0 0.1f
M1663 t576 nq12 t579 0 nch w=1u l=180n
M1664 t579 nw158 0 0 nch w=1u l=180n
M1665 t577 nq12 vdd vdd pch w=2u l=180n
M1666 t577 t576 vdd vdd pch w=2u l=180n
CT580 t580 0 0.1f
M1667 t577 nq12 t580 0 nch w=1u l=180n
M1668 t580 t576 0 0 nch w=1u l=180n
M1669 t578 nw158 vdd vdd pch w=2u l=180n
M1670 t578 t576 vdd vdd pch w=2u l=180n
CT581 t581 0 0.1f
M1671 t578 nw158 t581 0 nch w=1u l=180n
M1672 t581 t576 0 0 nch w=1u l=180n
M1673 nw256 t577 vdd vdd pch w=2u l=180n
M1674 nw256 t578 vdd vdd pch w=2u l=180n
CT582 t582 0 0.1f
M1675 nw256 t577 t582 0 nch w=1u l=180n
M1676 t582 t578 0 0 nch w=1u l=180n
Cnw256 nw256 0 2f
M1677 nw257 nq13 vdd vdd pch w=2u l=180n
M1678 nw257 nw160 vdd vdd pch w=2u l=180n
CT583 t583 0 0.1f
M1679 nw257 nq13 t583 0 nch w=1u l=180n
M1680 t583 nw160 0 0 nch w=1u l=180n
Cnw257 nw257 0 2f
M1681 nw258 nq14 0 0 nch w=1u l=180n
M1682 nw258 nw162 0 0 nch w=1u l=180n
CT584 t584 0 0.1f
M1683 t584 nq14 vdd vdd pch w=2u l=180n
M1684 nw258 nw162 t584 vdd pch w=2u l=180n
Cnw258 nw258 0 2f
CT585 t585 0 0.1f
M1685 t585 nq15 vdd vdd pch w=2u l=180n
M1686 t585 nw164 vdd vdd pch w=2u l=180n
CT586 t586 0 0.1f
M1687 t585 nq15 t586 0 nch w=1u l=180n
M1688 t586 nw164 0 0 nch w=1u l=180n
M1689 nw259 t585 vdd vdd pch w=2u l=180n
M1690 nw259 t585 0 0 nch w=1u l=180n
Cnw259 nw259 0 2f
CT587 t587 0 0.1f
M1691 t587 nq16 0 0 nch w=1u l=180n
M1692 t587 nw166 0 0 nch w=1u l=180n
CT588 t588 0 0.1f
M1693 t588 nq16 vdd vdd pch w=2u l=180n
M1694 t587 nw166 t588 vdd pch w=2u l=180n
M1695 nw260 t587 vdd vdd pch w=2u l=180n
M1696 nw260 t587 0 0 nch w=1u l=180n
Cnw260 nw260 0 2f
CT589 t589 0 0.1f
CT590 t590 0 0.1f
CT591 t591 0 0.1f
M1697 t589 nq17 vdd vdd pch w=2u l=180n
M1698 t589 nw168 vdd vdd pch w=2u l=180n
CT592 t592 0 0.1f
M1699 t589 nq17 t592 0 nch w=1u l=180n
M1700 t592 nw168 0 0 nch w=1u l=180n
M1701 t590 nq17 vdd vdd pch w=2u l=180n
M1702 t590 t589 vdd vdd pch w=2u l=180n
CT593 t593 0 0.1f
M1703 t590 nq17 t593 0 nch w=1u l=180n
M1704 t593 t589 0 0 nch w=1u l=180n
M1705 t591 nw168 vdd vdd pch w=2u l=180n
M1706 t591 t589 vdd vdd pch w=2u l=180n
CT594 t594 0 0.1f
M1707 t591 nw168 t594 0 nch w=1u l=180n
M1708 t594 t589 0 0 nch w=1u l=180n
M1709 nw261 t590 vdd vdd pch w=2u l=180n
M1710 nw261 t591 vdd vdd pch w=2u l=180n
CT595 t595 0 0.1f
M1711 nw261 t590 t595 0 nch w=1u l=180n
M1712 t595 t591 0 0 nch w=1u l=180n
Cnw261 nw261 0 2f
M1713 nw262 nq18 vdd vdd pch w=2u l=180n
M1714 nw262 nw170 vdd vdd pch w=2u l=180n
CT596 t596 0 0.1f
M1715 nw262 nq18 t596 0 nch w=1u l=180n
M1716 t596 nw170 0 0 nch w=1u l=180n
Cnw262 nw262 0 2f
M1717 nw263 ni0 0 0 nch w=1u l=180n
M1718 nw263 nw172 0 0 nch w=1u l=180n
CT597 t597 0 0.1f
M1719 t597 ni0 vdd vdd pch w=2u l=180n
M1720 nw263 nw172 t597 vdd pch w=2u l=180n
Cnw263 nw263 0 2f
CT598 t598 0 0.1f
M1721 t598 ni1 vdd vdd pch w=2u l=180n
M1722 t598 nw174 vdd vdd pch w=2u l=180n
CT599 t599 0 0.1f
M1723 t598 ni1 t599 0 nch w=1u l=180n
M1724 t599 nw174 0 0 nch w=1u l=180n
M1725 nw264 t598 vdd vdd pch w=2u l=180n
M1726 nw264 t598 0 0 nch w=1u l=180n
Cnw264 nw264 0 2f
CT600 t600 0 0.1f
M1727 t600 ni2 0 0 nch w=1u l=180n
M1728 t600 nw176 0 0 nch w=1u l=180n
CT601 t601 0 0.1f
M1729 t601 ni2 vdd vdd pch w=2u l=180n
M1730 t600 nw176 t601 vdd pch w=2u l=180n
M1731 nw265 t600 vdd vdd pch w=2u l=180n
M1732 nw265 t600 0 0 nch w=1u l=180n
Cnw265 nw265 0 2f
CT602 t602 0 0.1f
CT603 t603 0 0.1f
CT604 t604 0 0.1f
M1733 t602 ni3 vdd vdd pch w=2u l=180n
M1734 t602 nw178 vdd vdd pch w=2u l=180n
CT605 t605 0 0.1f
M1735 t602 ni3 t605 0 nch w=1u l=180n
M1736 t605 nw178 0 0 nch w=1u l=180n
M1737 t603 ni3 vdd vdd pch w=2u l=180n
M1738 t603 t602 vdd vdd pch w=2u l=180n
CT606 t606 0 0.1f
M1739 t603 ni3 t606 0 nch w=1u l=180n
M1740 t606 t602 0 0 nch w=1u l=180n
M1741 t604 nw178 vdd vdd pch w=2u l=180n
M1742 t604 t602 vdd vdd pch w=2u l=180n
CT607 t607 0 0.1f
M1743 t604 nw178 t607 0 nch w=1u l=180n
M1744 t607 t602 0 0 nch w=1u l=180n
M1745 nw266 t603 vdd vdd pch w=2u l=180n
M1746 nw266 t604 vdd vdd pch w=2u l=180n
CT608 t608 0 0.1f
M1747 nw266 t603 t608 0 nch w=1u l=180n
M1748 t608 t604 0 0 nch w=1u l=180n
Cnw266 nw266 0 2f
M1749 nw267 ni4 vdd vdd pch w=2u l=180n
M1750 nw267 nw180 vdd vdd pch w=2u l=180n
CT609 t609 0 0.1f
M1751 nw267 ni4 t609 0 nch w=1u l=180n
M1752 t609 nw180 0 0 nch w=1u l=180n
Cnw267 nw267 0 2f
M1753 nw268 ni5 0 0 nch w=1u l=180n
M1754 nw268 nw182 0 0 nch w=1u l=180n
CT610 t610 0 0.1f
M1755 t610 ni5 vdd vdd pch w=2u l=180n
M1756 nw268 nw182 t610 vdd pch w=2u l=180n
Cnw268 nw268 0 2f
CT611 t611 0 0.1f
M1757 t611 ni6 vdd vdd pch w=2u l=180n
M1758 t611 nw184 vdd vdd pch w=2u l=180n
CT612 t612 0 0.1f
M1759 t611 ni6 t612 0 nch w=1u l=180n
M1760 t612 nw184 0 0 nch w=1u l=180n
M1761 nw269 t611 vdd vdd pch w=2u l=180n
M1762 nw269 t611 0 0 nch w=1u l=180n
Cnw269 nw269 0 2f
CT613 t613 0 0.1f
M1763 t613 ni7 0 0 nch w=1u l=180n
M1764 t613 nw186 0 0 nch w=1u l=180n
CT614 t614 0 0.1f
M1765 t614 ni7 vdd vdd pch w=2u l=180n
M1766 t613 nw186 t614 vdd pch w=2u l=180n
M1767 nw270 t613 vdd vdd pch w=2u l=180n
M1768 nw270 t613 0 0 nch w=1u l=180n
Cnw270 nw270 0 2f
CT615 t615 0 0.1f
CT616 t616 0 0.1f
CT617 t617 0 0.1f
M1769 t615 ni8 vdd vdd pch w=2u l=180n
M1770 t615 nw188 vdd vdd pch w=2u l=180n
CT618 t618 0 0.1f
M1771 t615 ni8 t618 0 nch w=1u l=180n
M1772 t618 nw188 0 0 nch w=1u l=180n
M1773 t616 ni8 vdd vdd pch w=2u l=180n
M1774 t616 t615 vdd vdd pch w=2u l=180n
CT619 t619 0 0.1f
M1775 t616 ni8 t619 0 nch w=1u l=180n
M1776 t619 t615 0 0 nch w=1u l=180n
M1777 t617 nw188 vdd vdd pch w=2u l=180n
M1778 t617 t615 vdd vdd pch w=2u l=180n
CT620 t620 0 0.1f
M1779 t617 nw188 t620 0 nch w=1u l=180n
M1780 t620 t615 0 0 nch w=1u l=180n
M1781 nw271 t616 vdd vdd pch w=2u l=180n
M1782 nw271 t617 vdd vdd pch w=2u l=180n
CT621 t621 0 0.1f
M1783 nw271 t616 t621 0 nch w=1u l=180n
M1784 t621 t617 0 0 nch w=1u l=180n
Cnw271 nw271 0 2f
M1785 nw272 nw77 vdd vdd pch w=2u l=180n
M1786 nw272 nw190 vdd vdd pch w=2u l=180n
CT622 t622 0 0.1f
M1787 nw272 nw77 t622 0 nch w=1u l=180n
M1788 t622 nw190 0 0 nch w=1u l=180n
Cnw272 nw272 0 2f
M1789 nw273 nw78 0 0 nch w=1u l=180n
M1790 nw273 nw192 0 0 nch w=1u l=180n
CT623 t623 0 0.1f
M1791 t623 nw78 vdd vdd pch w=2u l=180n
M1792 nw273 nw192 t623 vdd pch w=2u l=180n
Cnw273 nw273 0 2f
CT624 t624 0 0.1f
M1793 t624 nw79 vdd vdd pch w=2u l=180n
M1794 t624 nw194 vdd vdd pch w=2u l=180n
CT625 t625 0 0.1f
M1795 t624 nw79 t625 0 nch w=1u l=180n
M1796 t625 nw194 0 0 nch w=1u l=180n
M1797 nw274 t624 vdd vdd pch w=2u l=180n
M1798 nw274 t624 0 0 nch w=1u l=180n
Cnw274 nw274 0 2f
CT626 t626 0 0.1f
M1799 t626 nw80 0 0 nch w=1u l=180n
M1800 t626 nw196 0 0 nch w=1u l=180n
CT627 t627 0 0.1f
M1801 t627 nw80 vdd vdd pch w=2u l=180n
M1802 t626 nw196 t627 vdd pch w=2u l=180n
M1803 nw275 t626 vdd vdd pch w=2u l=180n
M1804 nw275 t626 0 0 nch w=1u l=180n
Cnw275 nw275 0 2f
CT628 t628 0 0.1f
CT629 t629 0 0.1f
CT630 t630 0 0.1f
M1805 t628 nw81 vdd vdd pch w=2u l=180n
M1806 t628 nw198 vdd vdd pch w=2u l=180n
CT631 t631 0 0.1f
M1807 t628 nw81 t631 0 nch w=1u l=180n
M1808 t631 nw198 0 0 nch w=1u l=180n
M1809 t629 nw81 vdd vdd pch w=2u l=180n
M1810 t629 t628 vdd vdd pch w=2u l=180n
CT632 t632 0 0.1f
M1811 t629 nw81 t632 0 nch w=1u l=180n
M1812 t632 t628 0 0 nch w=1u l=180n
M1813 t630 nw198 vdd vdd pch w=2u l=180n
M1814 t630 t628 vdd vdd pch w=2u l=180n
CT633 t633 0 0.1f
M1815 t630 nw198 t633 0 nch w=1u l=180n
M1816 t633 t628 0 0 nch w=1u l=180n
M1817 nw276 t629 vdd vdd pch w=2u l=180n
M1818 nw276 t630 vdd vdd pch w=2u l=180n
CT634 t634 0 0.1f
M1819 nw276 t629 t634 0 nch w=1u l=180n
M1820 t634 t630 0 0 nch w=1u l=180n
Cnw276 nw276 0 2f
M1821 nw277 nw82 vdd vdd pch w=2u l=180n
M1822 nw277 nw200 vdd vdd pch w=2u l=180n
CT635 t635 0 0.1f
M1823 nw277 nw82 t635 0 nch w=1u l=180n
M1824 t635 nw200 0 0 nch w=1u l=180n
Cnw277 nw277 0 2f
M1825 nw278 nw83 0 0 nch w=1u l=180n
M1826 nw278 nw202 0 0 nch w=1u l=180n
CT636 t636 0 0.1f
M1827 t636 nw83 vdd vdd pch w=2u l=180n
M1828 nw278 nw202 t636 vdd pch w=2u l=180n
Cnw278 nw278 0 2f
CT637 t637 0 0.1f
M1829 t637 nw84 vdd vdd pch w=2u l=180n
M1830 t637 nw204 vdd vdd pch w=2u l=180n
CT638 t638 0 0.1f
M1831 t637 nw84 t638 0 nch w=1u l=180n
M1832 t638 nw204 0 0 nch w=1u l=180n
M1833 nw279 t637 vdd vdd pch w=2u l=180n
M1834 nw279 t637 0 0 nch w=1u l=180n
Cnw279 nw279 0 2f
CT639 t639 0 0.1f
M1835 t639 nw85 0 0 nch w=1u l=180n
M1836 t639 nw206 0 0 nch w=1u l=180n
CT640 t640 0 0.1f
M1837 t640 nw85 vdd vdd pch w=2u l=180n
M1838 t639 nw206 t640 vdd pch w=2u l=180n
M1839 nw280 t639 vdd vdd pch w=2u l=180n
M1840 nw280 t639 0 0 nch w=1u l=180n
Cnw280 nw280 0 2f
CT641 t641 0 0.1f
CT642 t642 0 0.1f
CT643 t643 0 0.1f
M1841 t641 nw86 vdd vdd pch w=2u l=180n
M1842 t641 nw208 vdd vdd pch w=2u l=180n
CT644 t644 0 0.1f
M1843 t641 nw86 t644 0 nch w=1u l=180n
M1844 t644 nw208 0 0 nch w=1u l=180n
M1845 t642 nw86 vdd vdd pch w=2u l=180n
M1846 t642 t641 vdd vdd pch w=2u l=180n
CT645 t645 0 0.1f
M1847 t642 nw86 t645 0 nch w=1u l=180n
M1848 t645 t641 0 0 nch w=1u l=180n
M1849 t643 nw208 vdd vdd pch w=2u l=180n
M1850 t643 t641 vdd vdd pch w=2u l=180n
CT646 t646 0 0.1f
M1851 t643 nw208 t646 0 nch w=1u l=180n
M1852 t646 t641 0 0 nch w=1u l=180n
M1853 nw281 t642 vdd vdd pch w=2u l=180n
M1854 nw281 t643 vdd vdd pch w=2u l=180n
CT647 t647 0 0.1f
M1855 nw281 t642 t647 0 nch w=1u l=180n
M1856 t647 t643 0 0 nch w=1u l=180n
Cnw281 nw281 0 2f
M1857 nw282 nw87 vdd vdd pch w=2u l=180n
M1858 nw282 nw210 vdd vdd pch w=2u l=180n
CT648 t648 0 0.1f
M1859 nw282 nw87 t648 0 nch w=1u l=180n
M1860 t648 nw210 0 0 nch w=1u l=180n
Cnw282 nw282 0 2f
M1861 nw283 nw88 0 0 nch w=1u l=180n
M1862 nw283 nw212 0 0 nch w=1u l=180n
CT649 t649 0 0.1f
M1863 t649 nw88 vdd vdd pch w=2u l=180n
M1864 nw283 nw212 t649 vdd pch w=2u l=180n
Cnw283 nw283 0 2f
CT650 t650 0 0.1f
M1865 t650 nw89 vdd vdd pch w=2u l=180n
M1866 t650 nw214 vdd vdd pch w=2u l=180n
CT651 t651 0 0.1f
M1867 t650 nw89 t651 0 nch w=1u l=180n
M1868 t651 nw214 0 0 nch w=1u l=180n
M1869 nw284 t650 vdd vdd pch w=2u l=180n
M1870 nw284 t650 0 0 nch w=1u l=180n
Cnw284 nw284 0 2f
CT652 t652 0 0.1f
M1871 t652 nw90 0 0 nch w=1u l=180n
M1872 t652 nw216 0 0 nch w=1u l=180n
CT653 t653 0 0.1f
M1873 t653 nw90 vdd vdd pch w=2u l=180n
M1874 t652 nw216 t653 vdd pch w=2u l=180n
M1875 nw285 t652 vdd vdd pch w=2u l=180n
M1876 nw285 t652 0 0 nch w=1u l=180n
Cnw285 nw285 0 2f
CT654 t654 0 0.1f
CT655 t655 0 0.1f
CT656 t656 0 0.1f
M1877 t654 nw91 vdd vdd pch w=2u l=180n
M1878 t654 nw218 vdd vdd pch w=2u l=180n
CT657 t657 0 0.1f
M1879 t654 nw91 t657 0 nch w=1u l=180n
M1880 t657 nw218 0 0 nch w=1u l=180n
M1881 t655 nw91 vdd vdd pch w=2u l=180n
M1882 t655 t654 vdd vdd pch w=2u l=180n
CT658 t658 0 0.1f
M1883 t655 nw91 t658 0 nch w=1u l=180n
M1884 t658 t654 0 0 nch w=1u l=180n
M1885 t656 nw218 vdd vdd pch w=2u l=180n
M1886 t656 t654 vdd vdd pch w=2u l=180n
CT659 t659 0 0.1f
M1887 t656 nw218 t659 0 nch w=1u l=180n
M1888 t659 t654 0 0 nch w=1u l=180n
M1889 nw286 t655 vdd vdd pch w=2u l=180n
M1890 nw286 t656 vdd vdd pch w=2u l=180n
CT660 t660 0 0.1f
M1891 nw286 t655 t660 0 nch w=1u l=180n
M1892 t660 t656 0 0 nch w=1u l=180n
Cnw286 nw286 0 2f
M1893 nw287 nw92 vdd vdd pch w=2u l=180n
M1894 nw287 nw220 vdd vdd pch w=2u l=180n
CT661 t661 0 0.1f
M1895 nw287 nw92 t661 0 nch w=1u l=180n
M1896 t661 nw220 0 0 nch w=1u l=180n
Cnw287 nw287 0 2f
M1897 nw288 nw93 0 0 nch w=1u l=180n
M1898 nw288 nw222 0 0 nch w=1u l=180n
CT662 t662 0 0.1f
M1899 t662 nw93 vdd vdd pch w=2u l=180n
M1900 nw288 nw222 t662 vdd pch w=2u l=180n
Cnw288 nw288 0 2f
CT663 t663 0 0.1f
M1901 t663 nw94 vdd vdd pch w=2u l=180n
M1902 t663 nw224 vdd vdd pch w=2u l=180n
CT664 t664 0 0.1f
M1903 t663 nw94 t664 0 nch w=1u l=180n
M1904 t664 nw224 0 0 nch w=1u l=180n
M1905 nw289 t663 vdd vdd pch w=2u l=180n
M1906 nw289 t663 0 0 nch w=1u l=180n
Cnw289 nw289 0 2f
CT665 t665 0 0.1f
M1907 t665 nw95 0 0 nch w=1u l=180n
M1908 t665 nw226 0 0 nch w=1u l=180n
CT666 t666 0 0.1f
M1909 t666 nw95 vdd vdd pch w=2u l=180n
M1910 t665 nw226 t666 vdd pch w=2u l=180n
M1911 nw290 t665 vdd vdd pch w=2u l=180n
M1912 nw290 t665 0 0 nch w=1u l=180n
Cnw290 nw290 0 2f
CT667 t667 0 0.1f
CT668 t668 0 0.1f
CT669 t669 0 0.1f
M1913 t667 nw96 vdd vdd pch w=2u l=180n
M1914 t667 nw228 vdd vdd pch w=2u l=180n
CT670 t670 0 0.1f
M1915 t667 nw96 t670 0 nch w=1u l=180n
M1916 t670 nw228 0 0 nch w=1u l=180n
M1917 t668 nw96 vdd vdd pch w=2u l=180n
M1918 t668 t667 vdd vdd pch w=2u l=180n
CT671 t671 0 0.1f
M1919 t668 nw96 t671 0 nch w=1u l=180n
M1920 t671 t667 0 0 nch w=1u l=180n
M1921 t669 nw228 vdd vdd pch w=2u l=180n
M1922 t669 t667 vdd vdd pch w=2u l=180n
CT672 t672 0 0.1f
M1923 t669 nw228 t672 0 nch w=1u l=180n
M1924 t672 t667 0 0 nch w=1u l=180n
M1925 nw291 t668 vdd vdd pch w=2u l=180n
M1926 nw291 t669 vdd vdd pch w=2u l=180n
CT673 t673 0 0.1f
M1927 nw291 t668 t673 0 nch w=1u l=180n
M1928 t673 t669 0 0 nch w=1u l=180n
Cnw291 nw291 0 2f
M1929 nw292 nw97 vdd vdd pch w=2u l=180n
M1930 nw292 nw230 vdd vdd pch w=2u l=180n
CT674 t674 0 0.1f
M1931 nw292 nw97 t674 0 nch w=1u l=180n
M1932 t674 nw230 0 0 nch w=1u l=180n
Cnw292 nw292 0 2f
M1933 nw293 nw98 0 0 nch w=1u l=180n
M1934 nw293 nw232 0 0 nch w=1u l=180n
CT675 t675 0 0.1f
M1935 t675 nw98 vdd vdd pch w=2u l=180n
M1936 nw293 nw232 t675 vdd pch w=2u l=180n
Cnw293 nw293 0 2f
CT676 t676 0 0.1f
M1937 t676 nw99 vdd vdd pch w=2u l=180n
M1938 t676 nw234 vdd vdd pch w=2u l=180n
CT677 t677 0 0.1f
M1939 t676 nw99 t677 0 nch w=1u l=180n
M1940 t677 nw234 0 0 nch w=1u l=180n
M1941 nw294 t676 vdd vdd pch w=2u l=180n
M1942 nw294 t676 0 0 nch w=1u l=180n
Cnw294 nw294 0 2f
CT678 t678 0 0.1f
M1943 t678 nw100 0 0 nch w=1u l=180n
M1944 t678 nw236 0 0 nch w=1u l=180n
CT679 t679 0 0.1f
M1945 t679 nw100 vdd vdd pch w=2u l=180n
M1946 t678 nw236 t679 vdd pch w=2u l=180n
M1947 nw295 t678 vdd vdd pch w=2u l=180n
M1948 nw295 t678 0 0 nch w=1u l=180n
Cnw295 nw295 0 2f
CT680 t680 0 0.1f
CT681 t681 0 0.1f
CT682 t682 0 0.1f
M1949 t680 nw101 vdd vdd pch w=2u l=180n
M1950 t680 nw238 vdd vdd pch w=2u l=180n
CT683 t683 0 0.1f
M1951 t680 nw101 t683 0 nch w=1u l=180n
M1952 t683 nw238 0 0 nch w=1u l=180n
M1953 t681 nw101 vdd vdd pch w=2u l=180n
M1954 t681 t680 vdd vdd pch w=2u l=180n
CT684 t684 0 0.1f
M1955 t681 nw101 t684 0 nch w=1u l=180n
M1956 t684 t680 0 0 nch w=1u l=180n
M1957 t682 nw238 vdd vdd pch w=2u l=180n
M1958 t682 t680 vdd vdd pch w=2u l=180n
CT685 t685 0 0.1f
M1959 t682 nw238 t685 0 nch w=1u l=180n
M1960 t685 t680 0 0 nch w=1u l=180n
M1961 nw296 t681 vdd vdd pch w=2u l=180n
M1962 nw296 t682 vdd vdd pch w=2u l=180n
CT686 t686 0 0.1f
M1963 nw296 t681 t686 0 nch w=1u l=180n
M1964 t686 t682 0 0 nch w=1u l=180n
Cnw296 nw296 0 2f
M1965 nw297 nw102 vdd vdd pch w=2u l=180n
M1966 nw297 nw240 vdd vdd pch w=2u l=180n
CT687 t687 0 0.1f
M1967 nw297 nw102 t687 0 nch w=1u l=180n
M1968 t687 nw240 0 0 nch w=1u l=180n
Cnw297 nw297 0 2f
M1969 nw298 nw103 0 0 nch w=1u l=180n
M1970 nw298 nw242 0 0 nch w=1u l=180n
CT688 t688 0 0.1f
M1971 t688 nw103 vdd vdd pch w=2u l=180n
M1972 nw298 nw242 t688 vdd pch w=2u l=180n
Cnw298 nw298 0 2f
CT689 t689 0 0.1f
M1973 t689 nw104 vdd vdd pch w=2u l=180n
M1974 t689 nw244 vdd vdd pch w=2u l=180n
CT690 t690 0 0.1f
M1975 t689 nw104 t690 0 nch w=1u l=180n
M1976 t690 nw244 0 0 nch w=1u l=180n
M1977 nw299 t689 vdd vdd pch w=2u l=180n
M1978 nw299 t689 0 0 nch w=1u l=180n
Cnw299 nw299 0 2f
CT691 t691 0 0.1f
M1979 t691 nw105 0 0 nch w=1u l=180n
M1980 t691 nw246 0 0 nch w=1u l=180n
CT692 t692 0 0.1f
M1981 t692 nw105 vdd vdd pch w=2u l=180n
M1982 t691 nw246 t692 vdd pch w=2u l=180n
M1983 nw300 t691 vdd vdd pch w=2u l=180n
M1984 nw300 t691 0 0 nch w=1u l=180n
Cnw300 nw300 0 2f
CT693 t693 0 0.1f
CT694 t694 0 0.1f
CT695 t695 0 0.1f
M1985 t693 nw106 vdd vdd pch w=2u l=180n
M1986 t693 nw248 vdd vdd pch w=2u l=180n
CT696 t696 0 0.1f
M1987 t693 nw106 t696 0 nch w=1u l=180n
M1988 t696 nw248 0 0 nch w=1u l=180n
M1989 t694 nw106 vdd vdd pch w=2u l=180n
M1990 t694 t693 vdd vdd pch w=2u l=180n
CT697 t697 0 0.1f
M1991 t694 nw106 t697 0 nch w=1u l=180n
M1992 t697 t693 0 0 nch w=1u l=180n
M1993 t695 nw248 vdd vdd pch w=2u l=180n
M1994 t695 t693 vdd vdd pch w=2u l=180n
CT698 t698 0 0.1f
M1995 t695 nw248 t698 0 nch w=1u l=180n
M1996 t698 t693 0 0 nch w=1u l=180n
M1997 nw301 t694 vdd vdd pch w=2u l=180n
M1998 nw301 t695 vdd vdd pch w=2u l=180n
CT699 t699 0 0.1f
M1999 nw301 t694 t699 0 nch w=1u l=180n
M2000 t699 t695 0 0 nch w=1u l=180n
Cnw301 nw301 0 2f
M2001 nw302 nw107 vdd vdd pch w=2u l=180n
M2002 nw302 nw250 vdd vdd pch w=2u l=180n
CT700 t700 0 0.1f
M2003 nw302 nw107 t700 0 nch w=1u l=180n
M2004 t700 nw250 0 0 nch w=1u l=180n
Cnw302 nw302 0 2f
M2005 nw303 nw108 0 0 nch w=1u l=180n
M2006 nw303 nw252 0 0 nch w=1u l=180n
CT701 t701 0 0.1f
M2007 t701 nw108 vdd vdd pch w=2u l=180n
M2008 nw303 nw252 t701 vdd pch w=2u l=180n
Cnw303 nw303 0 2f
CT702 t702 0 0.1f
M2009 t702 nw109 vdd vdd pch w=2u l=180n
M2010 t702 nw254 vdd vdd pch w=2u l=180n
CT703 t703 0 0.1f
M2011 t702 nw109 t703 0 nch w=1u l=180n
M2012 t703 nw254 0 0 nch w=1u l=180n
M2013 nw304 t702 vdd vdd pch w=2u l=180n
M2014 nw304 t702 0 0 nch w=1u l=180n
Cnw304 nw304 0 2f
CT704 t704 0 0.1f
M2015 t704 nw110 0 0 nch w=1u l=180n
M2016 t704 nw256 0 0 nch w=1u l=180n
CT705 t705 0 0.1f
M2017 t705 nw110 vdd vdd pch w=2u l=180n
M2018 t704 nw256 t705 vdd pch w=2u l=180n
M2019 nw305 t704 vdd vdd pch w=2u l=180n
M2020 nw305 t704 0 0 nch w=1u l=180n
Cnw305 nw305 0 2f
CT706 t706 0 0.1f
CT707 t707 0 0.1f
CT708 t708 0 0.1f
M2021 t706 nw111 vdd vdd pch w=2u l=180n
M2022 t706 nw258 vdd vdd pch w=2u l=180n
CT709 t709 0 0.1f
M2023 t706 nw111 t709 0 nch w=1u l=180n
M2024 t709 nw258 0 0 nch w=1u l=180n
M2025 t707 nw111 vdd vdd pch w=2u l=180n
M2026 t707 t706 vdd vdd pch w=2u l=180n
CT710 t710 0 0.1f
M2027 t707 nw111 t710 0 nch w=1u l=180n
M2028 t710 t706 0 0 nch w=1u l=180n
M2029 t708 nw258 vdd vdd pch w=2u l=180n
M2030 t708 t706 vdd vdd pch w=2u l=180n
CT711 t711 0 0.1f
M2031 t708 nw258 t711 0 nch w=1u l=180n
M2032 t711 t706 0 0 nch w=1u l=180n
M2033 nw306 t707 vdd vdd pch w=2u l=180n
M2034 nw306 t708 vdd vdd pch w=2u l=180n
CT712 t712 0 0.1f
M2035 nw306 t707 t712 0 nch w=1u l=180n
M2036 t712 t708 0 0 nch w=1u l=180n
Cnw306 nw306 0 2f
M2037 nw307 nw112 vdd vdd pch w=2u l=180n
M2038 nw307 nw260 vdd vdd pch w=2u l=180n
CT713 t713 0 0.1f
M2039 nw307 nw112 t713 0 nch w=1u l=180n
M2040 t713 nw260 0 0 nch w=1u l=180n
Cnw307 nw307 0 2f
M2041 nw308 nw113 0 0 nch w=1u l=180n
M2042 nw308 nw262 0 0 nch w=1u l=180n
CT714 t714 0 0.1f
M2043 t714 nw113 vdd vdd pch w=2u l=180n
M2044 nw308 nw262 t714 vdd pch w=2u l=180n
Cnw308 nw308 0 2f
CT715 t715 0 0.1f
M2045 t715 nw114 vdd vdd pch w=2u l=180n
M2046 t715 nw264 vdd vdd pch w=2u l=180n
CT716 t716 0 0.1f
M2047 t715 nw114 t716 0 nch w=1u l=180n
M2048 t716 nw264 0 0 nch w=1u l=180n
M2049 nw309 t715 vdd vdd pch w=2u l=180n
M2050 nw309 t715 0 0 nch w=1u l=180n
Cnw309 nw309 0 2f
CT717 t717 0 0.1f
M2051 t717 nw115 0 0 nch w=1u l=180n
M2052 t717 nw266 0 0 nch w=1u l=180n
CT718 t718 0 0.1f
M2053 t718 nw115 vdd vdd pch w=2u l=180n
M2054 t717 nw266 t718 vdd pch w=2u l=180n
M2055 nw310 t717 vdd vdd pch w=2u l=180n
M2056 nw310 t717 0 0 nch w=1u l=180n
Cnw310 nw310 0 2f
CT719 t719 0 0.1f
CT720 t720 0 0.1f
CT721 t721 0 0.1f
M2057 t719 nw116 vdd vdd pch w=2u l=180n
M2058 t719 nw268 vdd vdd pch w=2u l=180n
CT722 t722 0 0.1f
M2059 t719 nw116 t722 0 nch w=1u l=180n
M2060 t722 nw268 0 0 nch w=1u l=180n
M2061 t720 nw116 vdd vdd pch w=2u l=180n
M2062 t720 t719 vdd vdd pch w=2u l=180n
CT723 t723 0 0.1f
M2063 t720 nw116 t723 0 nch w=1u l=180n
M2064 t723 t719 0 0 nch w=1u l=180n
M2065 t721 nw268 vdd vdd pch w=2u l=180n
M2066 t721 t719 vdd vdd pch w=2u l=180n
CT724 t724 0 0.1f
M2067 t721 nw268 t724 0 nch w=1u l=180n
M2068 t724 t719 0 0 nch w=1u l=180n
M2069 nw311 t720 vdd vdd pch w=2u l=180n
M2070 nw311 t721 vdd vdd pch w=2u l=180n
CT725 t725 0 0.1f
M2071 nw311 t720 t725 0 nch w=1u l=180n
M2072 t725 t721 0 0 nch w=1u l=180n
Cnw311 nw311 0 2f
M2073 nw312 nw117 vdd vdd pch w=2u l=180n
M2074 nw312 nw270 vdd vdd pch w=2u l=180n
CT726 t726 0 0.1f
M2075 nw312 nw117 t726 0 nch w=1u l=180n
M2076 t726 nw270 0 0 nch w=1u l=180n
Cnw312 nw312 0 2f
M2077 nw313 nw118 0 0 nch w=1u l=180n
M2078 nw313 nw272 0 0 nch w=1u l=180n
CT727 t727 0 0.1f
M2079 t727 nw118 vdd vdd pch w=2u l=180n
M2080 nw313 nw272 t727 vdd pch w=2u l=180n
Cnw313 nw313 0 2f
CT728 t728 0 0.1f
M2081 t728 nw119 vdd vdd pch w=2u l=180n
M2082 t728 nw274 vdd vdd pch w=2u l=180n
CT729 t729 0 0.1f
M2083 t728 nw119 t729 0 nch w=1u l=180n
M2084 t729 nw274 0 0 nch w=1u l=180n
M2085 nw314 t728 vdd vdd pch w=2u l=180n
M2086 nw314 t728 0 0 nch w=1u l=180n
Cnw314 nw314 0 2f
CT730 t730 0 0.1f
M2087 t730 nw120 0 0 nch w=1u l=180n
M2088 t730 nw276 0 0 nch w=1u l=180n
CT731 t731 0 0.1f
M2089 t731 nw120 vdd vdd pch w=2u l=180n
M2090 t730 nw276 t731 vdd pch w=2u l=180n
M2091 nw315 t730 vdd vdd pch w=2u l=180n
M2092 nw315 t730 0 0 nch w=1u l=180n
Cnw315 nw315 0 2f
CT732 t732 0 0.1f
CT733 t733 0 0.1f
CT734 t734 0 0.1f
M2093 t732 nw121 vdd vdd pch w=2u l=180n
M2094 t732 nw278 vdd vdd pch w=2u l=180n
CT735 t735 0 0.1f
M2095 t732 nw121 t735 0 nch w=1u l=180n
M2096 t735 nw278 0 0 nch w=1u l=180n
M2097 t733 nw121 vdd vdd pch w=2u l=180n
M2098 t733 t732 vdd vdd pch w=2u l=180n
CT736 t736 0 0.1f
M2099 t733 nw121 t736 0 nch w=1u l=180n
M2100 t736 t732 0 0 nch w=1u l=180n
M2101 t734 nw278 vdd vdd pch w=2u l=180n
M2102 t734 t732 vdd vdd pch w=2u l=180n
CT737 t737 0 0.1f
M2103 t734 nw278 t737 0 nch w=1u l=180n
M2104 t737 t732 0 0 nch w=1u l=180n
M2105 nw316 t733 vdd vdd pch w=2u l=180n
M2106 nw316 t734 vdd vdd pch w=2u l=180n
CT738 t738 0 0.1f
M2107 nw316 t733 t738 0 nch w=1u l=180n
M2108 t738 t734 0 0 nch w=1u l=180n
Cnw316 nw316 0 2f
M2109 nw317 nw122 vdd vdd pch w=2u l=180n
M2110 nw317 nw280 vdd vdd pch w=2u l=180n
CT739 t739 0 0.1f
M2111 nw317 nw122 t739 0 nch w=1u l=180n
M2112 t739 nw280 0 0 nch w=1u l=180n
Cnw317 nw317 0 2f
M2113 nw318 nw123 0 0 nch w=1u l=180n
M2114 nw318 nw282 0 0 nch w=1u l=180n
CT740 t740 0 0.1f
M2115 t740 nw123 vdd vdd pch w=2u l=180n
M2116 nw318 nw282 t740 vdd pch w=2u l=180n
Cnw318 nw318 0 2f
CT741 t741 0 0.1f
M2117 t741 nw124 vdd vdd pch w=2u l=180n
M2118 t741 nw284 vdd vdd pch w=2u l=180n
CT742 t742 0 0.1f
M2119 t741 nw124 t742 0 nch w=1u l=180n
M2120 t742 nw284 0 0 nch w=1u l=180n
M2121 nw319 t741 vdd vdd pch w=2u l=180n
M2122 nw319 t741 0 0 nch w=1u l=180n
Cnw319 nw319 0 2f
CT743 t743 0 0.1f
M2123 t743 nw125 0 0 nch w=1u l=180n
M2124 t743 nw286 0 0 nch w=1u l=180n
CT744 t744 0 0.1f
M2125 t744 nw125 vdd vdd pch w=2u l=180n
M2126 t743 nw286 t744 vdd pch w=2u l=180n
M2127 nw320 t743 vdd vdd pch w=2u l=180n
M2128 nw320 t743 0 0 nch w=1u l=180n
Cnw320 nw320 0 2f
CT745 t745 0 0.1f
CT746 t746 0 0.1f
CT747 t747 0 0.1f
M2129 t745 nw126 vdd vdd pch w=2u l=180n
M2130 t745 nw288 vdd vdd pch w=2u l=180n
CT748 t748 0 0.1f
M2131 t745 nw126 t748 0 nch w=1u l=180n
M2132 t748 nw288 0 0 nch w=1u l=180n
M2133 t746 nw126 vdd vdd pch w=2u l=180n
M2134 t746 t745 vdd vdd pch w=2u l=180n
CT749 t749 0 0.1f
M2135 t746 nw126 t749 0 nch w=1u l=180n
M2136 t749 t745 0 0 nch w=1u l=180n
M2137 t747 nw288 vdd vdd pch w=2u l=180n
M2138 t747 t745 vdd vdd pch w=2u l=180n
CT750 t750 0 0.1f
M2139 t747 nw288 t750 0 nch w=1u l=180n
M2140 t750 t745 0 0 nch w=1u l=180n
M2141 nw321 t746 vdd vdd pch w=2u l=180n
M2142 nw321 t747 vdd vdd pch w=2u l=180n
CT751 t751 0 0.1f
M2143 nw321 t746 t751 0 nch w=1u l=180n
M2144 t751 t747 0 0 nch w=1u l=180n
Cnw321 nw321 0 2f
M2145 nw322 nw127 vdd vdd pch w=2u l=180n
M2146 nw322 nw290 vdd vdd pch w=2u l=180n
CT752 t752 0 0.1f
M2147 nw322 nw127 t752 0 nch w=1u l=180n
M2148 t752 nw290 0 0 nch w=1u l=180n
Cnw322 nw322 0 2f
M2149 nw323 nw128 0 0 nch w=1u l=180n
M2150 nw323 nw292 0 0 nch w=1u l=180n
CT753 t753 0 0.1f
M2151 t753 nw128 vdd vdd pch w=2u l=180n
M2152 nw323 nw292 t753 vdd pch w=2u l=180n
Cnw323 nw323 0 2f
CT754 t754 0 0.1f
M2153 t754 nw129 vdd vdd pch w=2u l=180n
M2154 t754 nw294 vdd vdd pch w=2u l=180n
CT755 t755 0 0.1f
M2155 t754 nw129 t755 0 nch w=1u l=180n
M2156 t755 nw294 0 0 nch w=1u l=180n
M2157 nw324 t754 vdd vdd pch w=2u l=180n
M2158 nw324 t754 0 0 nch w=1u l=180n
Cnw324 nw324 0 2f
CT756 t756 0 0.1f
M2159 t756 nw130 0 0 nch w=1u l=180n
M2160 t756 nw296 0 0 nch w=1u l=180n
CT757 t757 0 0.1f
M2161 t757 nw130 vdd vdd pch w=2u l=180n
M2162 t756 nw296 t757 vdd pch w=2u l=180n
M2163 nw325 t756 vdd vdd pch w=2u l=180n
M2164 nw325 t756 0 0 nch w=1u l=180n
Cnw325 nw325 0 2f
CT758 t758 0 0.1f
CT759 t759 0 0.1f
CT760 t760 0 0.1f
M2165 t758 nw131 vdd vdd pch w=2u l=180n
M2166 t758 nw298 vdd vdd pch w=2u l=180n
CT761 t761 0 0.1f
M2167 t758 nw131 t761 0 nch w=1u l=180n
M2168 t761 nw298 0 0 nch w=1u l=180n
M2169 t759 nw131 vdd vdd pch w=2u l=180n
M2170 t759 t758 vdd vdd pch w=2u l=180n
CT762 t762 0 0.1f
M2171 t759 nw131 t762 0 nch w=1u l=180n
M2172 t762 t758 0 0 nch w=1u l=180n
M2173 t760 nw298 vdd vdd pch w=2u l=180n
M2174 t760 t758 vdd vdd pch w=2u l=180n
CT763 t763 0 0.1f
M2175 t760 nw298 t763 0 nch w=1u l=180n
M2176 t763 t758 0 0 nch w=1u l=180n
M2177 nw326 t759 vdd vdd pch w=2u l=180n
M2178 nw326 t760 vdd vdd pch w=2u l=180n
CT764 t764 0 0.1f
M2179 nw326 t759 t764 0 nch w=1u l=180n
M2180 t764 t760 0 0 nch w=1u l=180n
Cnw326 nw326 0 2f
M2181 nw327 nw132 vdd vdd pch w=2u l=180n
M2182 nw327 nw300 vdd vdd pch w=2u l=180n
CT765 t765 0 0.1f
M2183 nw327 nw132 t765 0 nch w=1u l=180n
M2184 t765 nw300 0 0 nch w=1u l=180n
Cnw327 nw327 0 2f
M2185 nw328 nw133 0 0 nch w=1u l=180n
M2186 nw328 nw302 0 0 nch w=1u l=180n
CT766 t766 0 0.1f
M2187 t766 nw133 vdd vdd pch w=2u l=180n
M2188 nw328 nw302 t766 vdd pch w=2u l=180n
Cnw328 nw328 0 2f
CT767 t767 0 0.1f
M2189 t767 nw134 vdd vdd pch w=2u l=180n
M2190 t767 nw304 vdd vdd pch w=2u l=180n
CT768 t768 0 0.1f
M2191 t767 nw134 t768 0 nch w=1u l=180n
M2192 t768 nw304 0 0 nch w=1u l=180n
M2193 nw329 t767 vdd vdd pch w=2u l=180n
M2194 nw329 t767 0 0 nch w=1u l=180n
Cnw329 nw329 0 2f
CT769 t769 0 0.1f
M2195 t769 nw135 0 0 nch w=1u l=180n
M2196 t769 nw306 0 0 nch w=1u l=180n
CT770 t770 0 0.1f
M2197 t770 nw135 vdd vdd pch w=2u l=180n
M2198 t769 nw306 t770 vdd pch w=2u l=180n
M2199 nw330 t769 vdd vdd pch w=2u l=180n
M2200 nw330 t769 0 0 nch w=1u l=180n
Cnw330 nw330 0 2f
CT771 t771 0 0.1f
CT772 t772 0 0.1f
CT773 t773 0 0.1f
M2201 t771 nw136 vdd vdd pch w=2u l=180n
M2202 t771 nw308 vdd vdd pch w=2u l=180n
CT774 t774 0 0.1f
M2203 t771 nw136 t774 0 nch w=1u l=180n
M2204 t774 nw308 0 0 nch w=1u l=180n
M2205 t772 nw136 vdd vdd pch w=2u l=180n
M2206 t772 t771 vdd vdd pch w=2u l=180n
CT775 t775 0 0.1f
M2207 t772 nw136 t775 0 nch w=1u l=180n
M2208 t775 t771 0 0 nch w=1u l=180n
M2209 t773 nw308 vdd vdd pch w=2u l=180n
M2210 t773 t771 vdd vdd pch w=2u l=180n
CT776 t776 0 0.1f
M2211 t773 nw308 t776 0 nch w=1u l=180n
M2212 t776 t771 0 0 nch w=1u l=180n
M2213 nw331 t772 vdd vdd pch w=2u l=180n
M2214 nw331 t773 vdd vdd pch w=2u l=180n
CT777 t777 0 0.1f
M2215 nw331 t772 t777 0 nch w=1u l=180n
M2216 t777 t773 0 0 nch w=1u l=180n
Cnw331 nw331 0 2f
M2217 nw332 nw137 vdd vdd pch w=2u l=180n
M2218 nw332 nw310 vdd vdd pch w=2u l=180n
CT778 t778 0 0.1f
M2219 nw332 nw137 t778 0 nch w=1u l=180n
M2220 t778 nw310 0 0 nch w=1u l=180n
Cnw332 nw332 0 2f
M2221 nw333 nw138 0 0 nch w=1u l=180n
M2222 nw333 nw312 0 0 nch w=1u l=180n
CT779 t779 0 0.1f
M2223 t779 nw138 vdd vdd pch w=2u l=180n
M2224 nw333 nw312 t779 vdd pch w=2u l=180n
Cnw333 nw333 0 2f
CT780 t780 0 0.1f
M2225 t780 nw139 vdd vdd pch w=2u l=180n
M2226 t780 nw314 vdd vdd pch w=2u l=180n
CT781 t781 0 0.1f
M2227 t780 nw139 t781 0 nch w=1u l=180n
M2228 t781 nw314 0 0 nch w=1u l=180n
M2229 nw334 t780 vdd vdd pch w=2u l=180n
M2230 nw334 t780 0 0 nch w=1u l=180n
Cnw334 nw334 0 2f
CT782 t782 0 0.1f
M2231 t782 nw140 0 0 nch w=1u l=180n
M2232 t782 nw316 0 0 nch w=1u l=180n
CT783 t783 0 0.1f
M2233 t783 nw140 vdd vdd pch w=2u l=180n
M2234 t782 nw316 t783 vdd pch w=2u l=180n
M2235 nw335 t782 vdd vdd pch w=2u l=180n
M2236 nw335 t782 0 0 nch w=1u l=180n
Cnw335 nw335 0 2f
CT784 t784 0 0.1f
CT785 t785 0 0.1f
CT786 t786 0 0.1f
M2237 t784 nw141 vdd vdd pch w=2u l=180n
M2238 t784 nw318 vdd vdd pch w=2u l=180n
CT787 t787 0 0.1f
M2239 t784 nw141 t787 0 nch w=1u l=180n
M2240 t787 nw318 0 0 nch w=1u l=180n
M2241 t785 nw141 vdd vdd pch w=2u l=180n
M2242 t785 t784 vdd vdd pch w=2u l=180n
CT788 t788 0 0.1f
M2243 t785 nw141 t788 0 nch w=1u l=180n
M2244 t788 t784 0 0 nch w=1u l=180n
M2245 t786 nw318 vdd vdd pch w=2u l=180n
M2246 t786 t784 vdd vdd pch w=2u l=180n
CT789 t789 0 0.1f
M2247 t786 nw318 t789 0 nch w=1u l=180n
M2248 t789 t784 0 0 nch w=1u l=180n
M2249 nw336 t785 vdd vdd pch w=2u l=180n
M2250 nw336 t786 vdd vdd pch w=2u l=180n
CT790 t790 0 0.1f
M2251 nw336 t785 t790 0 nch w=1u l=180n
M2252 t790 t786 0 0 nch w=1u l=180n
Cnw336 nw336 0 2f
M2253 nw337 nw142 vdd vdd pch w=2u l=180n
M2254 nw337 nw320 vdd vdd pch w=2u l=180n
CT791 t791 0 0.1f
M2255 nw337 nw142 t791 0 nch w=1u l=180n
M2256 t791 nw320 0 0 nch w=1u l=180n
Cnw337 nw337 0 2f
M2257 nw338 nw143 0 0 nch w=1u l=180n
M2258 nw338 nw322 0 0 nch w=1u l=180n
CT792 t792 0 0.1f
M2259 t792 nw143 vdd vdd pch w=2u l=180n
M2260 nw338 nw322 t792 vdd pch w=2u l=180n
Cnw338 nw338 0 2f
CT793 t793 0 0.1f
M2261 t793 nw144 vdd vdd pch w=2u l=180n
M2262 t793 nw324 vdd vdd pch w=2u l=180n
CT794 t794 0 0.1f
M2263 t793 nw144 t794 0 nch w=1u l=180n
M2264 t794 nw324 0 0 nch w=1u l=180n
M2265 nw339 t793 vdd vdd pch w=2u l=180n
M2266 nw339 t793 0 0 nch w=1u l=180n
Cnw339 nw339 0 2f
CT795 t795 0 0.1f
M2267 t795 nw145 0 0 nch w=1u l=180n
M2268 t795 nw326 0 0 nch w=1u l=180n
CT796 t796 0 0.1f
M2269 t796 nw145 vdd vdd pch w=2u l=180n
M2270 t795 nw326 t796 vdd pch w=2u l=180n
M2271 nw340 t795 vdd vdd pch w=2u l=180n
M2272 nw340 t795 0 0 nch w=1u l=180n
Cnw340 nw340 0 2f
CT797 t797 0 0.1f
CT798 t798 0 0.1f
CT799 t799 0 0.1f
M2273 t797 nw146 vdd vdd pch w=2u l=180n
M2274 t797 nw328 vdd vdd pch w=2u l=180n
CT800 t800 0 0.1f
M2275 t797 nw146 t800 0 nch w=1u l=180n
M2276 t800 nw328 0 0 nch w=1u l=180n
M2277 t798 nw146 vdd vdd pch w=2u l=180n
M2278 t798 t797 vdd vdd pch w=2u l=180n
CT801 t801 0 0.1f
M2279 t798 nw146 t801 0 nch w=1u l=180n
M2280 t801 t797 0 0 nch w=1u l=180n
M2281 t799 nw328 vdd vdd pch w=2u l=180n
M2282 t799 t797 vdd vdd pch w=2u l=180n
CT802 t802 0 0.1f
M2283 t799 nw328 t802 0 nch w=1u l=180n
M2284 t802 t797 0 0 nch w=1u l=180n
M2285 nw341 t798 vdd vdd pch w=2u l=180n
M2286 nw341 t799 vdd vdd pch w=2u l=180n
CT803 t803 0 0.1f
M2287 nw341 t798 t803 0 nch w=1u l=180n
M2288 t803 t799 0 0 nch w=1u l=180n
Cnw341 nw341 0 2f
M2289 nw342 nw147 vdd vdd pch w=2u l=180n
M2290 nw342 nw330 vdd vdd pch w=2u l=180n
CT804 t804 0 0.1f
M2291 nw342 nw147 t804 0 nch w=1u l=180n
M2292 t804 nw330 0 0 nch w=1u l=180n
Cnw342 nw342 0 2f
M2293 nw343 nw148 0 0 nch w=1u l=180n
M2294 nw343 nw332 0 0 nch w=1u l=180n
CT805 t805 0 0.1f
M2295 t805 nw148 vdd vdd pch w=2u l=180n
M2296 nw343 nw332 t805 vdd pch w=2u l=180n
Cnw343 nw343 0 2f
CT806 t806 0 0.1f
M2297 t806 nw149 vdd vdd pch w=2u l=180n
M2298 t806 nw334 vdd vdd pch w=2u l=180n
CT807 t807 0 0.1f
M2299 t806 nw149 t807 0 nch w=1u l=180n
M2300 t807 nw334 0 0 nch w=1u l=180n
M2301 nw344 t806 vdd vdd pch w=2u l=180n
M2302 nw344 t806 0 0 nch w=1u l=180n
Cnw344 nw344 0 2f
CT808 t808 0 0.1f
M2303 t808 nw150 0 0 nch w=1u l=180n
M2304 t808 nw336 0 0 nch w=1u l=180n
CT809 t809 0 0.1f
M2305 t809 nw150 vdd vdd pch w=2u l=180n
M2306 t808 nw336 t809 vdd pch w=2u l=180n
M2307 nw345 t808 vdd vdd pch w=2u l=180n
M2308 nw345 t808 0 0 nch w=1u l=180n
Cnw345 nw345 0 2f
CT810 t810 0 0.1f
CT811 t811 0 0.1f
CT812 t812 0 0.1f
M2309 t810 nw151 vdd vdd pch w=2u l=180n
M2310 t810 nw338 vdd vdd pch w=2u l=180n
CT813 t813 0 0.1f
M2311 t810 nw151 t813 0 nch w=1u l=180n
M2312 t813 nw338 0 0 nch w=1u l=180n
M2313 t811 nw151 vdd vdd pch w=2u l=180n
M2314 t811 t810 vdd vdd pch w=2u l=180n
CT814 t814 0 0.1f
M2315 t811 nw151 t814 0 nch w=1u l=180n
M2316 t814 t810 0 0 nch w=1u l=180n
M2317 t812 nw338 vdd vdd pch w=2u l=180n
M2318 t812 t810 vdd vdd pch w=2u l=180n
CT815 t815 0 0.1f
M2319 t812 nw338 t815 0 nch w=1u l=180n
M2320 t815 t810 0 0 nch w=1u l=180n
M2321 nw346 t811 vdd vdd pch w=2u l=180n
M2322 nw346 t812 vdd vdd pch w=2u l=180n
CT816 t816 0 0.1f
M2323 nw346 t811 t816 0 nch w=1u l=180n
M2324 t816 t812 0 0 nch w=1u l=180n
Cnw346 nw346 0 2f
M2325 nw347 nw152 vdd vdd pch w=2u l=180n
M2326 nw347 nw340 vdd vdd pch w=2u l=180n
CT817 t817 0 0.1f
M2327 nw347 nw152 t817 0 nch w=1u l=180n
M2328 t817 nw340 0 0 nch w=1u l=180n
Cnw347 nw347 0 2f
M2329 nw348 nw153 0 0 nch w=1u l=180n
M2330 nw348 nw342 0 0 nch w=1u l=180n
CT818 t818 0 0.1f
M2331 t818 nw153 vdd vdd pch w=2u l=180n
M2332 nw348 nw342 t818 vdd pch w=2u l=180n
Cnw348 nw348 0 2f
CT819 t819 0 0.1f
M2333 t819 nw154 vdd vdd pch w=2u l=180n
M2334 t819 nw344 vdd vdd pch w=2u l=180n
CT820 t820 0 0.1f
M2335 t819 nw154 t820 0 nch w=1u l=180n
M2336 t820 nw344 0 0 nch w=1u l=180n
M2337 nw349 t819 vdd vdd pch w=2u l=180n
M2338 nw349 t819 0 0 nch w=1u l=180n
Cnw349 nw349 0 2f
CT821 t821 0 0.1f
M2339 t821 nw155 0 0 nch w=1u l=180n
M2340 t821 nw346 0 0 nch w=1u l=180n
CT822 t822 0 0.1f
M2341 t822 nw155 vdd vdd pch w=2u l=180n
M2342 t821 nw346 t822 vdd pch w=2u l=180n
M2343 nw350 t821 vdd vdd pch w=2u l=180n
M2344 nw350 t821 0 0 nch w=1u l=180n
Cnw350 nw350 0 2f
CT823 t823 0 0.1f
CT824 t824 0 0.1f
CT825 t825 0 0.1f
M2345 t823 nw156 vdd vdd pch w=2u l=180n
M2346 t823 nw348 vdd vdd pch w=2u l=180n
CT826 t826 0 0.1f
M2347 t823 nw156 t826 0 nch w=1u l=180n
M2348 t826 nw348 0 0 nch w=1u l=180n
M2349 t824 nw156 vdd vdd pch w=2u l=180n
M2350 t824 t823 vdd vdd pch w=2u l=180n
CT827 t827 0 0.1f
M2351 t824 nw156 t827 0 nch w=1u l=180n
M2352 t827 t823 0 0 nch w=1u l=180n
M2353 t825 nw348 vdd vdd pch w=2u l=180n
M2354 t825 t823 vdd vdd pch w=2u l=180n
CT828 t828 0 0.1f
M2355 t825 nw348 t828 0 nch w=1u l=180n
M2356 t828 t823 0 0 nch w=1u l=180n
M2357 nw351 t824 vdd vdd pch w=2u l=180n
M2358 nw351 t825 vdd vdd pch w=2u l=180n
CT829 t829 0 0.1f
M2359 nw351 t824 t829 0 nch w=1u l=180n
M2360 t829 t825 0 0 nch w=1u l=180n
Cnw351 nw351 0 2f
M2361 nw352 nw157 vdd vdd pch w=2u l=180n
M2362 nw352 nw350 vdd vdd pch w=2u l=180n
CT830 t830 0 0.1f
M2363 nw352 nw157 t830 0 nch w=1u l=180n
M2364 t830 nw350 0 0 nch w=1u l=180n
Cnw352 nw352 0 2f
M2365 nw353 nw158 0 0 nch w=1u l=180n
M2366 nw353 nw352 0 0 nch w=1u l=180n
CT831 t831 0 0.1f
M2367 t831 nw158 vdd vdd pch w=2u l=180n
M2368 nw353 nw352 t831 vdd pch w=2u l=180n
Cnw353 nw353 0 2f
CT832 t832 0 0.1f
M2369 t832 nw159 vdd vdd pch w=2u l=180n
M2370 t832 nq0 vdd vdd pch w=2u l=180n
CT833 t833 0 0.1f
M2371 t832 nw159 t833 0 nch w=1u l=180n
M2372 t833 nq0 0 0 nch w=1u l=180n
M2373 nw354 t832 vdd vdd pch w=2u l=180n
M2374 nw354 t832 0 0 nch w=1u l=180n
Cnw354 nw354 0 2f
CT834 t834 0 0.1f
M2375 t834 nw160 0 0 nch w=1u l=180n
M2376 t834 nq1 0 0 nch w=1u l=180n
CT835 t835 0 0.1f
M2377 t835 nw160 vdd vdd pch w=2u l=180n
M2378 t834 nq1 t835 vdd pch w=2u l=180n
M2379 nw355 t834 vdd vdd pch w=2u l=180n
M2380 nw355 t834 0 0 nch w=1u l=180n
Cnw355 nw355 0 2f
CT836 t836 0 0.1f
CT837 t837 0 0.1f
CT838 t838 0 0.1f
M2381 t836 nw161 vdd vdd pch w=2u l=180n
M2382 t836 nq2 vdd vdd pch w=2u l=180n
CT839 t839 0 0.1f
M2383 t836 nw161 t839 0 nch w=1u l=180n
M2384 t839 nq2 0 0 nch w=1u l=180n
M2385 t837 nw161 vdd vdd pch w=2u l=180n
M2386 t837 t836 vdd vdd pch w=2u l=180n
CT840 t840 0 0.1f
M2387 t837 nw161 t840 0 nch w=1u l=180n
M2388 t840 t836 0 0 nch w=1u l=180n
M2389 t838 nq2 vdd vdd pch w=2u l=180n
M2390 t838 t836 vdd vdd pch w=2u l=180n
CT841 t841 0 0.1f
M2391 t838 nq2 t841 0 nch w=1u l=180n
M2392 t841 t836 0 0 nch w=1u l=180n
M2393 nw356 t837 vdd vdd pch w=2u l=180n
M2394 nw356 t838 vdd vdd pch w=2u l=180n
CT842 t842 0 0.1f
M2395 nw356 t837 t842 0 nch w=1u l=180n
M2396 t842 t838 0 0 nch w=1u l=180n
Cnw356 nw356 0 2f
M2397 nw357 nw162 vdd vdd pch w=2u l=180n
M2398 nw357 nq3 vdd vdd pch w=2u l=180n
CT843 t843 0 0.1f
M2399 nw357 nw162 t843 0 nch w=1u l=180n
M2400 t843 nq3 0 0 nch w=1u l=180n
Cnw357 nw357 0 2f
M2401 nw358 nw163 0 0 nch w=1u l=180n
M2402 nw358 nq4 0 0 nch w=1u l=180n
CT844 t844 0 0.1f
M2403 t844 nw163 vdd vdd pch w=2u l=180n
M2404 nw358 nq4 t844 vdd pch w=2u l=180n
Cnw358 nw358 0 2f
CT845 t845 0 0.1f
M2405 t845 nw164 vdd vdd pch w=2u l=180n
M2406 t845 nq5 vdd vdd pch w=2u l=180n
CT846 t846 0 0.1f
M2407 t845 nw164 t846 0 nch w=1u l=180n
M2408 t846 nq5 0 0 nch w=1u l=180n
M2409 nw359 t845 vdd vdd pch w=2u l=180n
M2410 nw359 t845 0 0 nch w=1u l=180n
Cnw359 nw359 0 2f
CT847 t847 0 0.1f
M2411 t847 nw165 0 0 nch w=1u l=180n
M2412 t847 nq6 0 0 nch w=1u l=180n
CT848 t848 0 0.1f
M2413 t848 nw165 vdd vdd pch w=2u l=180n
M2414 t847 nq6 t848 vdd pch w=2u l=180n
M2415 nw360 t847 vdd vdd pch w=2u l=180n
M2416 nw360 t847 0 0 nch w=1u l=180n
Cnw360 nw360 0 2f
CT849 t849 0 0.1f
CT850 t850 0 0.1f
CT851 t851 0 0.1f
M2417 t849 nw166 vdd vdd pch w=2u l=180n
M2418 t849 nq7 vdd vdd pch w=2u l=180n
CT852 t852 0 0.1f
M2419 t849 nw166 t852 0 nch w=1u l=180n
M2420 t852 nq7 0 0 nch w=1u l=180n
M2421 t850 nw166 vdd vdd pch w=2u l=180n
M2422 t850 t849 vdd vdd pch w=2u l=180n
CT853 t853 0 0.1f
M2423 t850 nw166 t853 0 nch w=1u l=180n
M2424 t853 t849 0 0 nch w=1u l=180n
M2425 t851 nq7 vdd vdd pch w=2u l=180n
M2426 t851 t849 vdd vdd pch w=2u l=180n
CT854 t854 0 0.1f
M2427 t851 nq7 t854 0 nch w=1u l=180n
M2428 t854 t849 0 0 nch w=1u l=180n
M2429 nw361 t850 vdd vdd pch w=2u l=180n
M2430 nw361 t851 vdd vdd pch w=2u l=180n
CT855 t855 0 0.1f
M2431 nw361 t850 t855 0 nch w=1u l=180n
M2432 t855 t851 0 0 nch w=1u l=180n
Cnw361 nw361 0 2f
M2433 nw362 nw167 vdd vdd pch w=2u l=180n
M2434 nw362 nq8 vdd vdd pch w=2u l=180n
CT856 t856 0 0.1f
M2435 nw362 nw167 t856 0 nch w=1u l=180n
M2436 t856 nq8 0 0 nch w=1u l=180n
Cnw362 nw362 0 2f
M2437 nw363 nw168 0 0 nch w=1u l=180n
M2438 nw363 nq9 0 0 nch w=1u l=180n
CT857 t857 0 0.1f
M2439 t857 nw168 vdd vdd pch w=2u l=180n
M2440 nw363 nq9 t857 vdd pch w=2u l=180n
Cnw363 nw363 0 2f
CT858 t858 0 0.1f
M2441 t858 nw169 vdd vdd pch w=2u l=180n
M2442 t858 nq10 vdd vdd pch w=2u l=180n
CT859 t859 0 0.1f
M2443 t858 nw169 t859 0 nch w=1u l=180n
M2444 t859 nq10 0 0 nch w=1u l=180n
M2445 nw364 t858 vdd vdd pch w=2u l=180n
M2446 nw364 t858 0 0 nch w=1u l=180n
Cnw364 nw364 0 2f
CT860 t860 0 0.1f
M2447 t860 nw170 0 0 nch w=1u l=180n
M2448 t860 nq11 0 0 nch w=1u l=180n
CT861 t861 0 0.1f
M2449 t861 nw170 vdd vdd pch w=2u l=180n
M2450 t860 nq11 t861 vdd pch w=2u l=180n
M2451 nw365 t860 vdd vdd pch w=2u l=180n
M2452 nw365 t860 0 0 nch w=1u l=180n
Cnw365 nw365 0 2f
CT862 t862 0 0.1f
CT863 t863 0 0.1f
CT864 t864 0 0.1f
M2453 t862 nw171 vdd vdd pch w=2u l=180n
M2454 t862 nq12 vdd vdd pch w=2u l=180n
CT865 t865 0 0.1f
M2455 t862 nw171 t865 0 nch w=1u l=180n
M2456 t865 nq12 0 0 nch w=1u l=180n
M2457 t863 nw171 vdd vdd pch w=2u l=180n
M2458 t863 t862 vdd vdd pch w=2u l=180n
CT866 t866 0 0.1f
M2459 t863 nw171 t866 0 nch w=1u l=180n
M2460 t866 t862 0 0 nch w=1u l=180n
M2461 t864 nq12 vdd vdd pch w=2u l=180n
M2462 t864 t862 vdd vdd pch w=2u l=180n
CT867 t867 0 0.1f
M2463 t864 nq12 t867 0 nch w=1u l=180n
M2464 t867 t862 0 0 nch w=1u l=180n
M2465 nw366 t863 vdd vdd pch w=2u l=180n
M2466 nw366 t864 vdd vdd pch w=2u l=180n
CT868 t868 0 0.1f
M2467 nw366 t863 t868 0 nch w=1u l=180n
M2468 t868 t864 0 0 nch w=1u l=180n
Cnw366 nw366 0 2f
M2469 nw367 nw172 vdd vdd pch w=2u l=180n
M2470 nw367 nq13 vdd vdd pch w=2u l=180n
CT869 t869 0 0.1f
M2471 nw367 nw172 t869 0 nch w=1u l=180n
M2472 t869 nq13 0 0 nch w=1u l=180n
Cnw367 nw367 0 2f
M2473 nw368 nw173 0 0 nch w=1u l=180n
M2474 nw368 nq14 0 0 nch w=1u l=180n
CT870 t870 0 0.1f
M2475 t870 nw173 vdd vdd pch w=2u l=180n
M2476 nw368 nq14 t870 vdd pch w=2u l=180n
Cnw368 nw368 0 2f
CT871 t871 0 0.1f
M2477 t871 nw174 vdd vdd pch w=2u l=180n
M2478 t871 nq15 vdd vdd pch w=2u l=180n
CT872 t872 0 0.1f
M2479 t871 nw174 t872 0 nch w=1u l=180n
M2480 t872 nq15 0 0 nch w=1u l=180n
M2481 nw369 t871 vdd vdd pch w=2u l=180n
M2482 nw369 t871 0 0 nch w=1u l=180n
Cnw369 nw369 0 2f
CT873 t873 0 0.1f
M2483 t873 nw175 0 0 nch w=1u l=180n
M2484 t873 nq16 0 0 nch w=1u l=180n
CT874 t874 0 0.1f
M2485 t874 nw175 vdd vdd pch w=2u l=180n
M2486 t873 nq16 t874 vdd pch w=2u l=180n
M2487 nw370 t873 vdd vdd pch w=2u l=180n
M2488 nw370 t873 0 0 nch w=1u l=180n
Cnw370 nw370 0 2f
CT875 t875 0 0.1f
CT876 t876 0 0.1f
CT877 t877 0 0.1f
M2489 t875 nw176 vdd vdd pch w=2u l=180n
M2490 t875 nq17 vdd vdd pch w=2u l=180n
CT878 t878 0 0.1f
M2491 t875 nw176 t878 0 nch w=1u l=180n
M2492 t878 nq17 0 0 nch w=1u l=180n
M2493 t876 nw176 vdd vdd pch w=2u l=180n
M2494 t876 t875 vdd vdd pch w=2u l=180n
CT879 t879 0 0.1f
M2495 t876 nw176 t879 0 nch w=1u l=180n
M2496 t879 t875 0 0 nch w=1u l=180n
M2497 t877 nq17 vdd vdd pch w=2u l=180n
M2498 t877 t875 vdd vdd pch w=2u l=180n
CT880 t880 0 0.1f
M2499 t877 nq17 t880 0 nch w=1u l=180n
M2500 t880 t875 0 0 nch w=1u l=180n
M2501 nw371 t876 vdd vdd pch w=2u l=180n
M2502 nw371 t877 vdd vdd pch w=2u l=180n
CT881 t881 0 0.1f
M2503 nw371 t876 t881 0 nch w=1u l=180n
M2504 t881 t877 0 0 nch w=1u l=180n
Cnw371 nw371 0 2f
M2505 nw372 nw177 vdd vdd pch w=2u l=180n
M2506 nw372 nq18 vdd vdd pch w=2u l=180n
CT882 t882 0 0.1f
M2507 nw372 nw177 t882 0 nch w=1u l=180n
M2508 t882 nq18 0 0 nch w=1u l=180n
Cnw372 nw372 0 2f
M2509 nw373 nw178 0 0 nch w=1u l=180n
M2510 nw373 ni0 0 0 nch w=1u l=180n
CT883 t883 0 0.1f
M2511 t883 nw178 vdd vdd pch w=2u l=180n
M2512 nw373 ni0 t883 vdd pch w=2u l=180n
Cnw373 nw373 0 2f
CT884 t884 0 0.1f
M2513 t884 nw179 vdd vdd pch w=2u l=180n
M2514 t884 ni1 vdd vdd pch w=2u l=180n
CT885 t885 0 0.1f
M2515 t884 nw179 t885 0 nch w=1u l=180n
M2516 t885 ni1 0 0 nch w=1u l=180n
M2517 nw374 t884 vdd vdd pch w=2u l=180n
M2518 nw374 t884 0 0 nch w=1u l=180n
Cnw374 nw374 0 2f
CT886 t886 0 0.1f
M2519 t886 nw180 0 0 nch w=1u l=180n
M2520 t886 ni2 0 0 nch w=1u l=180n
CT887 t887 0 0.1f
M2521 t887 nw180 vdd vdd pch w=2u l=180n
M2522 t886 ni2 t887 vdd pch w=2u l=180n
M2523 nw375 t886 vdd vdd pch w=2u l=180n
M2524 nw375 t886 0 0 nch w=1u l=180n
Cnw375 nw375 0 2f
CT888 t888 0 0.1f
CT889 t889 0 0.1f
CT890 t890 0 0.1f
M2525 t888 nw181 vdd vdd pch w=2u l=180n
M2526 t888 ni3 vdd vdd pch w=2u l=180n
CT891 t891 0 0.1f
M2527 t888 nw181 t891 0 nch w=1u l=180n
M2528 t891 ni3 0 0 nch w=1u l=180n
M2529 t889 nw181 vdd vdd pch w=2u l=180n
M2530 t889 t888 vdd vdd pch w=2u l=180n
CT892 t892 0 0.1f
M2531 t889 nw181 t892 0 nch w=1u l=180n
M2532 t892 t888 0 0 nch w=1u l=180n
M2533 t890 ni3 vdd vdd pch w=2u l=180n
M2534 t890 t888 vdd vdd pch w=2u l=180n
CT893 t893 0 0.1f
M2535 t890 ni3 t893 0 nch w=1u l=180n
M2536 t893 t888 0 0 nch w=1u l=180n
M2537 nw376 t889 vdd vdd pch w=2u l=180n
M2538 nw376 t890 vdd vdd pch w=2u l=180n
CT894 t894 0 0.1f
M2539 nw376 t889 t894 0 nch w=1u l=180n
M2540 t894 t890 0 0 nch w=1u l=180n
Cnw376 nw376 0 2f
M2541 nw377 nw182 vdd vdd pch w=2u l=180n
M2542 nw377 ni4 vdd vdd pch w=2u l=180n
CT895 t895 0 0.1f
M2543 nw377 nw182 t895 0 nch w=1u l=180n
M2544 t895 ni4 0 0 nch w=1u l=180n
Cnw377 nw377 0 2f
M2545 nw378 nw183 0 0 nch w=1u l=180n
M2546 nw378 ni5 0 0 nch w=1u l=180n
CT896 t896 0 0.1f
M2547 t896 nw183 vdd vdd pch w=2u l=180n
M2548 nw378 ni5 t896 vdd pch w=2u l=180n
Cnw378 nw378 0 2f
CT897 t897 0 0.1f
M2549 t897 nw184 vdd vdd pch w=2u l=180n
M2550 t897 ni6 vdd vdd pch w=2u l=180n
CT898 t898 0 0.1f
M2551 t897 nw184 t898 0 nch w=1u l=180n
M2552 t898 ni6 0 0 nch w=1u l=180n
M2553 nw379 t897 vdd vdd pch w=2u l=180n
M2554 nw379 t897 0 0 nch w=1u l=180n
Cnw379 nw379 0 2f
CT899 t899 0 0.1f
M2555 t899 nw185 0 0 nch w=1u l=180n
M2556 t899 ni7 0 0 nch w=1u l=180n
CT900 t900 0 0.1f
M2557 t900 nw185 vdd vdd pch w=2u l=180n
M2558 t899 ni7 t900 vdd pch w=2u l=180n
M2559 nw380 t899 vdd vdd pch w=2u l=180n
M2560 nw380 t899 0 0 nch w=1u l=180n
Cnw380 nw380 0 2f
CT901 t901 0 0.1f
CT902 t902 0 0.1f
CT903 t903 0 0.1f
M2561 t901 nw186 vdd vdd pch w=2u l=180n
M2562 t901 ni8 vdd vdd pch w=2u l=180n
CT904 t904 0 0.1f
M2563 t901 nw186 t904 0 nch w=1u l=180n
M2564 t904 ni8 0 0 nch w=1u l=180n
M2565 t902 nw186 vdd vdd pch w=2u l=180n
M2566 t902 t901 vdd vdd pch w=2u l=180n
CT905 t905 0 0.1f
M2567 t902 nw186 t905 0 nch w=1u l=180n
M2568 t905 t901 0 0 nch w=1u l=180n
M2569 t903 ni8 vdd vdd pch w=2u l=180n
M2570 t903 t901 vdd vdd pch w=2u l=180n
CT906 t906 0 0.1f
M2571 t903 ni8 t906 0 nch w=1u l=180n
M2572 t906 t901 0 0 nch w=1u l=180n
M2573 nw381 t902 vdd vdd pch w=2u l=180n
M2574 nw381 t903 vdd vdd pch w=2u l=180n
CT907 t907 0 0.1f
M2575 nw381 t902 t907 0 nch w=1u l=180n
M2576 t907 t903 0 0 nch w=1u l=180n
Cnw381 nw381 0 2f
M2577 nw382 nw187 vdd vdd pch w=2u l=180n
M2578 nw382 nw77 vdd vdd pch w=2u l=180n
CT908 t908 0 0.1f
M2579 nw382 nw187 t908 0 nch w=1u l=180n
M2580 t908 nw77 0 0 nch w=1u l=180n
Cnw382 nw382 0 2f
M2581 nw383 nw188 0 0 nch w=1u l=180n
M2582 nw383 nw78 0 0 nch w=1u l=180n
CT909 t909 0 0.1f
M2583 t909 nw188 vdd vdd pch w=2u l=180n
M2584 nw383 nw78 t909 vdd pch w=2u l=180n
Cnw383 nw383 0 2f
CT910 t910 0 0.1f
M2585 t910 nw189 vdd vdd pch w=2u l=180n
M2586 t910 nw79 vdd vdd pch w=2u l=180n
CT911 t911 0 0.1f
M2587 t910 nw189 t911 0 nch w=1u l=180n
M2588 t911 nw79 0 0 nch w=1u l=180n
M2589 nw384 t910 vdd vdd pch w=2u l=180n
M2590 nw384 t910 0 0 nch w=1u l=180n
Cnw384 nw384 0 2f
CT912 t912 0 0.1f
M2591 t912 nw190 0 0 nch w=1u l=180n
M2592 t912 nw80 0 0 nch w=1u l=180n
CT913 t913 0 0.1f
M2593 t913 nw190 vdd vdd pch w=2u l=180n
M2594 t912 nw80 t913 vdd pch w=2u l=180n
M2595 nw385 t912 vdd vdd pch w=2u l=180n
M2596 nw385 t912 0 0 nch w=1u l=180n
Cnw385 nw385 0 2f
CT914 t914 0 0.1f
CT915 t915 0 0.1f
CT916 t916 0 0.1f
M2597 t914 nw191 vdd vdd pch w=2u l=180n
M2598 t914 nw81 vdd vdd pch w=2u l=180n
CT917 t917 0 0.1f
M2599 t914 nw191 t917 0 nch w=1u l=180n
M2600 t917 nw81 0 0 nch w=1u l=180n
M2601 t915 nw191 vdd vdd pch w=2u l=180n
M2602 t915 t914 vdd vdd pch w=2u l=180n
CT918 t918 0 0.1f
M2603 t915 nw191 t918 0 nch w=1u l=180n
M2604 t918 t914 0 0 nch w=1u l=180n
M2605 t916 nw81 vdd vdd pch w=2u l=180n
M2606 t916 t914 vdd vdd pch w=2u l=180n
CT919 t919 0 0.1f
M2607 t916 nw81 t919 0 nch w=1u l=180n
M2608 t919 t914 0 0 nch w=1u l=180n
M2609 nw386 t915 vdd vdd pch w=2u l=180n
M2610 nw386 t916 vdd vdd pch w=2u l=180n
CT920 t920 0 0.1f
M2611 nw386 t915 t920 0 nch w=1u l=180n
M2612 t920 t916 0 0 nch w=1u l=180n
Cnw386 nw386 0 2f
M2613 nw387 nw192 vdd vdd pch w=2u l=180n
M2614 nw387 nw82 vdd vdd pch w=2u l=180n
CT921 t921 0 0.1f
M2615 nw387 nw192 t921 0 nch w=1u l=180n
M2616 t921 nw82 0 0 nch w=1u l=180n
Cnw387 nw387 0 2f
M2617 nw388 nw193 0 0 nch w=1u l=180n
M2618 nw388 nw83 0 0 nch w=1u l=180n
CT922 t922 0 0.1f
M2619 t922 nw193 vdd vdd pch w=2u l=180n
M2620 nw388 nw83 t922 vdd pch w=2u l=180n
Cnw388 nw388 0 2f
CT923 t923 0 0.1f
M2621 t923 nw194 vdd vdd pch w=2u l=180n
M2622 t923 nw84 vdd vdd pch w=2u l=180n
CT924 t924 0 0.1f
M2623 t923 nw194 t924 0 nch w=1u l=180n
M2624 t924 nw84 0 0 nch w=1u l=180n
M2625 nw389 t923 vdd vdd pch w=2u l=180n
M2626 nw389 t923 0 0 nch w=1u l=180n
Cnw389 nw389 0 2f
CT925 t925 0 0.1f
M2627 t925 nw195 0 0 nch w=1u l=180n
M2628 t925 nw85 0 0 nch w=1u l=180n
CT926 t926 0 0.1f
M2629 t926 nw195 vdd vdd pch w=2u l=180n
M2630 t925 nw85 t926 vdd pch w=2u l=180n
M2631 nw390 t925 vdd vdd pch w=2u l=180n
M2632 nw390 t925 0 0 nch w=1u l=180n
Cnw390 nw390 0 2f
CT927 t927 0 0.1f
CT928 t928 0 0.1f
CT929 t929 0 0.1f
M2633 t927 nw196 vdd vdd pch w=2u l=180n
M2634 t927 nw86 vdd vdd pch w=2u l=180n
CT930 t930 0 0.1f
M2635 t927 nw196 t930 0 nch w=1u l=180n
M2636 t930 nw86 0 0 nch w=1u l=180n
M2637 t928 nw196 vdd vdd pch w=2u l=180n
M2638 t928 t927 vdd vdd pch w=2u l=180n
CT931 t931 0 0.1f
M2639 t928 nw196 t931 0 nch w=1u l=180n
M2640 t931 t927 0 0 nch w=1u l=180n
M2641 t929 nw86 vdd vdd pch w=2u l=180n
M2642 t929 t927 vdd vdd pch w=2u l=180n
CT932 t932 0 0.1f
M2643 t929 nw86 t932 0 nch w=1u l=180n
M2644 t932 t927 0 0 nch w=1u l=180n
M2645 nw391 t928 vdd vdd pch w=2u l=180n
M2646 nw391 t929 vdd vdd pch w=2u l=180n
CT933 t933 0 0.1f
M2647 nw391 t928 t933 0 nch w=1u l=180n
M2648 t933 t929 0 0 nch w=1u l=180n
Cnw391 nw391 0 2f
M2649 nw392 nw197 vdd vdd pch w=2u l=180n
M2650 nw392 nw87 vdd vdd pch w=2u l=180n
CT934 t934 0 0.1f
M2651 nw392 nw197 t934 0 nch w=1u l=180n
M2652 t934 nw87 0 0 nch w=1u l=180n
Cnw392 nw392 0 2f
M2653 nw393 nw198 0 0 nch w=1u l=180n
M2654 nw393 nw88 0 0 nch w=1u l=180n
CT935 t935 0 0.1f
M2655 t935 nw198 vdd vdd pch w=2u l=180n
M2656 nw393 nw88 t935 vdd pch w=2u l=180n
Cnw393 nw393 0 2f
CT936 t936 0 0.1f
M2657 t936 nw199 vdd vdd pch w=2u l=180n
M2658 t936 nw89 vdd vdd pch w=2u l=180n
CT937 t937 0 0.1f
M2659 t936 nw199 t937 0 nch w=1u l=180n
M2660 t937 nw89 0 0 nch w=1u l=180n
M2661 nw394 t936 vdd vdd pch w=2u l=180n
M2662 nw394 t936 0 0 nch w=1u l=180n
Cnw394 nw394 0 2f
CT938 t938 0 0.1f
M2663 t938 nw200 0 0 nch w=1u l=180n
M2664 t938 nw90 0 0 nch w=1u l=180n
CT939 t939 0 0.1f
M2665 t939 nw200 vdd vdd pch w=2u l=180n
M2666 t938 nw90 t939 vdd pch w=2u l=180n
M2667 nw395 t938 vdd vdd pch w=2u l=180n
M2668 nw395 t938 0 0 nch w=1u l=180n
Cnw395 nw395 0 2f
CT940 t940 0 0.1f
CT941 t941 0 0.1f
CT942 t942 0 0.1f
M2669 t940 nw201 vdd vdd pch w=2u l=180n
M2670 t940 nw91 vdd vdd pch w=2u l=180n
CT943 t943 0 0.1f
M2671 t940 nw201 t943 0 nch w=1u l=180n
M2672 t943 nw91 0 0 nch w=1u l=180n
M2673 t941 nw201 vdd vdd pch w=2u l=180n
M2674 t941 t940 vdd vdd pch w=2u l=180n
CT944 t944 0 0.1f
M2675 t941 nw201 t944 0 nch w=1u l=180n
M2676 t944 t940 0 0 nch w=1u l=180n
M2677 t942 nw91 vdd vdd pch w=2u l=180n
M2678 t942 t940 vdd vdd pch w=2u l=180n
CT945 t945 0 0.1f
M2679 t942 nw91 t945 0 nch w=1u l=180n
M2680 t945 t940 0 0 nch w=1u l=180n
M2681 nw396 t941 vdd vdd pch w=2u l=180n
M2682 nw396 t942 vdd vdd pch w=2u l=180n
CT946 t946 0 0.1f
M2683 nw396 t941 t946 0 nch w=1u l=180n
M2684 t946 t942 0 0 nch w=1u l=180n
Cnw396 nw396 0 2f
M2685 nw397 nw202 vdd vdd pch w=2u l=180n
M2686 nw397 nw92 vdd vdd pch w=2u l=180n
CT947 t947 0 0.1f
M2687 nw397 nw202 t947 0 nch w=1u l=180n
M2688 t947 nw92 0 0 nch w=1u l=180n
Cnw397 nw397 0 2f
M2689 nw398 nw203 0 0 nch w=1u l=180n
M2690 nw398 nw93 0 0 nch w=1u l=180n
CT948 t948 0 0.1f
M2691 t948 nw203 vdd vdd pch w=2u l=180n
M2692 nw398 nw93 t948 vdd pch w=2u l=180n
Cnw398 nw398 0 2f
CT949 t949 0 0.1f
M2693 t949 nw204 vdd vdd pch w=2u l=180n
M2694 t949 nw94 vdd vdd pch w=2u l=180n
CT950 t950 0 0.1f
M2695 t949 nw204 t950 0 nch w=1u l=180n
M2696 t950 nw94 0 0 nch w=1u l=180n
M2697 nw399 t949 vdd vdd pch w=2u l=180n
M2698 nw399 t949 0 0 nch w=1u l=180n
Cnw399 nw399 0 2f
CT951 t951 0 0.1f
M2699 t951 nw205 0 0 nch w=1u l=180n
M2700 t951 nw95 0 0 nch w=1u l=180n
CT952 t952 0 0.1f
M2701 t952 nw205 vdd vdd pch w=2u l=180n
M2702 t951 nw95 t952 vdd pch w=2u l=180n
M2703 nw400 t951 vdd vdd pch w=2u l=180n
M2704 nw400 t951 0 0 nch w=1u l=180n
Cnw400 nw400 0 2f
CT953 t953 0 0.1f
CT954 t954 0 0.1f
CT955 t955 0 0.1f
M2705 t953 nw206 vdd vdd pch w=2u l=180n
M2706 t953 nw96 vdd vdd pch w=2u l=180n
CT956 t956 0 0.1f
M2707 t953 nw206 t956 0 nch w=1u l=180n
M2708 t956 nw96 0 0 nch w=1u l=180n
M2709 t954 nw206 vdd vdd pch w=2u l=180n
M2710 t954 t953 vdd vdd pch w=2u l=180n
CT957 t957 0 0.1f
M2711 t954 nw206 t957 0 nch w=1u l=180n
M2712 t957 t953 0 0 nch w=1u l=180n
M2713 t955 nw96 vdd vdd pch w=2u l=180n
M2714 t955 t953 vdd vdd pch w=2u l=180n
CT958 t958 0 0.1f
M2715 t955 nw96 t958 0 nch w=1u l=180n
M2716 t958 t953 0 0 nch w=1u l=180n
M2717 nw401 t954 vdd vdd pch w=2u l=180n
M2718 nw401 t955 vdd vdd pch w=2u l=180n
CT959 t959 0 0.1f
M2719 nw401 t954 t959 0 nch w=1u l=180n
M2720 t959 t955 0 0 nch w=1u l=180n
Cnw401 nw401 0 2f
M2721 nw402 nw207 vdd vdd pch w=2u l=180n
M2722 nw402 nw97 vdd vdd pch w=2u l=180n
CT960 t960 0 0.1f
M2723 nw402 nw207 t960 0 nch w=1u l=180n
M2724 t960 nw97 0 0 nch w=1u l=180n
Cnw402 nw402 0 2f
M2725 nw403 nw208 0 0 nch w=1u l=180n
M2726 nw403 nw98 0 0 nch w=1u l=180n
CT961 t961 0 0.1f
M2727 t961 nw208 vdd vdd pch w=2u l=180n
M2728 nw403 nw98 t961 vdd pch w=2u l=180n
Cnw403 nw403 0 2f
CT962 t962 0 0.1f
M2729 t962 nw209 vdd vdd pch w=2u l=180n
M2730 t962 nw99 vdd vdd pch w=2u l=180n
CT963 t963 0 0.1f
M2731 t962 nw209 t963 0 nch w=1u l=180n
M2732 t963 nw99 0 0 nch w=1u l=180n
M2733 nw404 t962 vdd vdd pch w=2u l=180n
M2734 nw404 t962 0 0 nch w=1u l=180n
Cnw404 nw404 0 2f
CT964 t964 0 0.1f
M2735 t964 nw210 0 0 nch w=1u l=180n
M2736 t964 nw100 0 0 nch w=1u l=180n
CT965 t965 0 0.1f
M2737 t965 nw210 vdd vdd pch w=2u l=180n
M2738 t964 nw100 t965 vdd pch w=2u l=180n
M2739 nw405 t964 vdd vdd pch w=2u l=180n
M2740 nw405 t964 0 0 nch w=1u l=180n
Cnw405 nw405 0 2f
CT966 t966 0 0.1f
CT967 t967 0 0.1f
CT968 t968 0 0.1f
M2741 t966 nw211 vdd vdd pch w=2u l=180n
M2742 t966 nw101 vdd vdd pch w=2u l=180n
CT969 t969 0 0.1f
M2743 t966 nw211 t969 0 nch w=1u l=180n
M2744 t969 nw101 0 0 nch w=1u l=180n
M2745 t967 nw211 vdd vdd pch w=2u l=180n
M2746 t967 t966 vdd vdd pch w=2u l=180n
CT970 t970 0 0.1f
M2747 t967 nw211 t970 0 nch w=1u l=180n
M2748 t970 t966 0 0 nch w=1u l=180n
M2749 t968 nw101 vdd vdd pch w=2u l=180n
M2750 t968 t966 vdd vdd pch w=2u l=180n
CT971 t971 0 0.1f
M2751 t968 nw101 t971 0 nch w=1u l=180n
M2752 t971 t966 0 0 nch w=1u l=180n
M2753 nw406 t967 vdd vdd pch w=2u l=180n
M2754 nw406 t968 vdd vdd pch w=2u l=180n
CT972 t972 0 0.1f
M2755 nw406 t967 t972 0 nch w=1u l=180n
M2756 t972 t968 0 0 nch w=1u l=180n
Cnw406 nw406 0 2f
M2757 nw407 nw212 vdd vdd pch w=2u l=180n
M2758 nw407 nw102 vdd vdd pch w=2u l=180n
CT973 t973 0 0.1f
M2759 nw407 nw212 t973 0 nch w=1u l=180n
M2760 t973 nw102 0 0 nch w=1u l=180n
Cnw407 nw407 0 2f
M2761 nw408 nw213 0 0 nch w=1u l=180n
M2762 nw408 nw103 0 0 nch w=1u l=180n
CT974 t974 0 0.1f
M2763 t974 nw213 vdd vdd pch w=2u l=180n
M2764 nw408 nw103 t974 vdd pch w=2u l=180n
Cnw408 nw408 0 2f
CT975 t975 0 0.1f
M2765 t975 nw214 vdd vdd pch w=2u l=180n
M2766 t975 nw104 vdd vdd pch w=2u l=180n
CT976 t976 0 0.1f
M2767 t975 nw214 t976 0 nch w=1u l=180n
M2768 t976 nw104 0 0 nch w=1u l=180n
M2769 nw409 t975 vdd vdd pch w=2u l=180n
M2770 nw409 t975 0 0 nch w=1u l=180n
Cnw409 nw409 0 2f
CT977 t977 0 0.1f
M2771 t977 nw215 0 0 nch w=1u l=180n
M2772 t977 nw105 0 0 nch w=1u l=180n
CT978 t978 0 0.1f
M2773 t978 nw215 vdd vdd pch w=2u l=180n
M2774 t977 nw105 t978 vdd pch w=2u l=180n
M2775 nw410 t977 vdd vdd pch w=2u l=180n
M2776 nw410 t977 0 0 nch w=1u l=180n
Cnw410 nw410 0 2f
CT979 t979 0 0.1f
CT980 t980 0 0.1f
CT981 t981 0 0.1f
M2777 t979 nw216 vdd vdd pch w=2u l=180n
M2778 t979 nw106 vdd vdd pch w=2u l=180n
CT982 t982 0 0.1f
M2779 t979 nw216 t982 0 nch w=1u l=180n
M2780 t982 nw106 0 0 nch w=1u l=180n
M2781 t980 nw216 vdd vdd pch w=2u l=180n
M2782 t980 t979 vdd vdd pch w=2u l=180n
CT983 t983 0 0.1f
M2783 t980 nw216 t983 0 nch w=1u l=180n
M2784 t983 t979 0 0 nch w=1u l=180n
M2785 t981 nw106 vdd vdd pch w=2u l=180n
M2786 t981 t979 vdd vdd pch w=2u l=180n
CT984 t984 0 0.1f
M2787 t981 nw106 t984 0 nch w=1u l=180n
M2788 t984 t979 0 0 nch w=1u l=180n
M2789 nw411 t980 vdd vdd pch w=2u l=180n
M2790 nw411 t981 vdd vdd pch w=2u l=180n
CT985 t985 0 0.1f
M2791 nw411 t980 t985 0 nch w=1u l=180n
M2792 t985 t981 0 0 nch w=1u l=180n
Cnw411 nw411 0 2f
M2793 nw412 nw217 vdd vdd pch w=2u l=180n
M2794 nw412 nw107 vdd vdd pch w=2u l=180n
CT986 t986 0 0.1f
M2795 nw412 nw217 t986 0 nch w=1u l=180n
M2796 t986 nw107 0 0 nch w=1u l=180n
Cnw412 nw412 0 2f
M2797 nw413 nw218 0 0 nch w=1u l=180n
M2798 nw413 nw108 0 0 nch w=1u l=180n
CT987 t987 0 0.1f
M2799 t987 nw218 vdd vdd pch w=2u l=180n
M2800 nw413 nw108 t987 vdd pch w=2u l=180n
Cnw413 nw413 0 2f
CT988 t988 0 0.1f
M2801 t988 nw219 vdd vdd pch w=2u l=180n
M2802 t988 nw109 vdd vdd pch w=2u l=180n
CT989 t989 0 0.1f
M2803 t988 nw219 t989 0 nch w=1u l=180n
M2804 t989 nw109 0 0 nch w=1u l=180n
M2805 nw414 t988 vdd vdd pch w=2u l=180n
M2806 nw414 t988 0 0 nch w=1u l=180n
Cnw414 nw414 0 2f
CT990 t990 0 0.1f
M2807 t990 nw220 0 0 nch w=1u l=180n
M2808 t990 nw110 0 0 nch w=1u l=180n
CT991 t991 0 0.1f
M2809 t991 nw220 vdd vdd pch w=2u l=180n
M2810 t990 nw110 t991 vdd pch w=2u l=180n
M2811 nw415 t990 vdd vdd pch w=2u l=180n
M2812 nw415 t990 0 0 nch w=1u l=180n
Cnw415 nw415 0 2f
CT992 t992 0 0.1f
CT993 t993 0 0.1f
CT994 t994 0 0.1f
M2813 t992 nw221 vdd vdd pch w=2u l=180n
M2814 t992 nw111 vdd vdd pch w=2u l=180n
CT995 t995 0 0.1f
M2815 t992 nw221 t995 0 nch w=1u l=180n
M2816 t995 nw111 0 0 nch w=1u l=180n
M2817 t993 nw221 vdd vdd pch w=2u l=180n
M2818 t993 t992 vdd vdd pch w=2u l=180n
CT996 t996 0 0.1f
M2819 t993 nw221 t996 0 nch w=1u l=180n
M2820 t996 t992 0 0 nch w=1u l=180n
M2821 t994 nw111 vdd vdd pch w=2u l=180n
M2822 t994 t992 vdd vdd pch w=2u l=180n
CT997 t997 0 0.1f
M2823 t994 nw111 t997 0 nch w=1u l=180n
M2824 t997 t992 0 0 nch w=1u l=180n
M2825 nw416 t993 vdd vdd pch w=2u l=180n
M2826 nw416 t994 vdd vdd pch w=2u l=180n
CT998 t998 0 0.1f
M2827 nw416 t993 t998 0 nch w=1u l=180n
M2828 t998 t994 0 0 nch w=1u l=180n
Cnw416 nw416 0 2f
M2829 nw417 nw222 vdd vdd pch w=2u l=180n
M2830 nw417 nw112 vdd vdd pch w=2u l=180n
CT999 t999 0 0.1f
M2831 nw417 nw222 t999 0 nch w=1u l=180n
M2832 t999 nw112 0 0 nch w=1u l=180n
Cnw417 nw417 0 2f
M2833 nw418 nw223 0 0 nch w=1u l=180n
M2834 nw418 nw113 0 0 nch w=1u l=180n
CT1000 t1000 0 0.1f
M2835 t1000 nw223 vdd vdd pch w=2u l=180n
M2836 nw418 nw113 t1000 vdd pch w=2u l=180n
Cnw418 nw418 0 2f
CT1001 t1001 0 0.1f
M2837 t1001 nw224 vdd vdd pch w=2u l=180n
M2838 t1001 nw114 vdd vdd pch w=2u l=180n
CT1002 t1002 0 0.1f
M2839 t1001 nw224 t1002 0 nch w=1u l=180n
M2840 t1002 nw114 0 0 nch w=1u l=180n
M2841 nw419 t1001 vdd vdd pch w=2u l=180n
M2842 nw419 t1001 0 0 nch w=1u l=180n
Cnw419 nw419 0 2f
CT1003 t1003 0 0.1f
M2843 t1003 nw225 0 0 nch w=1u l=180n
M2844 t1003 nw115 0 0 nch w=1u l=180n
CT1004 t1004 0 0.1f
M2845 t1004 nw225 vdd vdd pch w=2u l=180n
M2846 t1003 nw115 t1004 vdd pch w=2u l=180n
M2847 nw420 t1003 vdd vdd pch w=2u l=180n
M2848 nw420 t1003 0 0 nch w=1u l=180n
Cnw420 nw420 0 2f
CT1005 t1005 0 0.1f
CT1006 t1006 0 0.1f
CT1007 t1007 0 0.1f
M2849 t1005 nw226 vdd vdd pch w=2u l=180n
M2850 t1005 nw116 vdd vdd pch w=2u l=180n
CT1008 t1008 0 0.1f
M2851 t1005 nw226 t1008 0 nch w=1u l=180n
M2852 t1008 nw116 0 0 nch w=1u l=180n
M2853 t1006 nw226 vdd vdd pch w=2u l=180n
M2854 t1006 t1005 vdd vdd pch w=2u l=180n
CT1009 t1009 0 0.1f
M2855 t1006 nw226 t1009 0 nch w=1u l=180n
M2856 t1009 t1005 0 0 nch w=1u l=180n
M2857 t1007 nw116 vdd vdd pch w=2u l=180n
M2858 t1007 t1005 vdd vdd pch w=2u l=180n
CT1010 t1010 0 0.1f
M2859 t1007 nw116 t1010 0 nch w=1u l=180n
M2860 t1010 t1005 0 0 nch w=1u l=180n
M2861 nw421 t1006 vdd vdd pch w=2u l=180n
M2862 nw421 t1007 vdd vdd pch w=2u l=180n
CT1011 t1011 0 0.1f
M2863 nw421 t1006 t1011 0 nch w=1u l=180n
M2864 t1011 t1007 0 0 nch w=1u l=180n
Cnw421 nw421 0 2f
M2865 nw422 nw227 vdd vdd pch w=2u l=180n
M2866 nw422 nw117 vdd vdd pch w=2u l=180n
CT1012 t1012 0 0.1f
M2867 nw422 nw227 t1012 0 nch w=1u l=180n
M2868 t1012 nw117 0 0 nch w=1u l=180n
Cnw422 nw422 0 2f
M2869 nw423 nw228 0 0 nch w=1u l=180n
M2870 nw423 nw118 0 0 nch w=1u l=180n
CT1013 t1013 0 0.1f
M2871 t1013 nw228 vdd vdd pch w=2u l=180n
M2872 nw423 nw118 t1013 vdd pch w=2u l=180n
Cnw423 nw423 0 2f
CT1014 t1014 0 0.1f
M2873 t1014 nw229 vdd vdd pch w=2u l=180n
M2874 t1014 nw119 vdd vdd pch w=2u l=180n
CT1015 t1015 0 0.1f
M2875 t1014 nw229 t1015 0 nch w=1u l=180n
M2876 t1015 nw119 0 0 nch w=1u l=180n
M2877 nw424 t1014 vdd vdd pch w=2u l=180n
M2878 nw424 t1014 0 0 nch w=1u l=180n
Cnw424 nw424 0 2f
CT1016 t1016 0 0.1f
M2879 t1016 nw230 0 0 nch w=1u l=180n
M2880 t1016 nw120 0 0 nch w=1u l=180n
CT1017 t1017 0 0.1f
M2881 t1017 nw230 vdd vdd pch w=2u l=180n
M2882 t1016 nw120 t1017 vdd pch w=2u l=180n
M2883 nw425 t1016 vdd vdd pch w=2u l=180n
M2884 nw425 t1016 0 0 nch w=1u l=180n
Cnw425 nw425 0 2f
CT1018 t1018 0 0.1f
CT1019 t1019 0 0.1f
CT1020 t1020 0 0.1f
M2885 t1018 nw231 vdd vdd pch w=2u l=180n
M2886 t1018 nw121 vdd vdd pch w=2u l=180n
CT1021 t1021 0 0.1f
M2887 t1018 nw231 t1021 0 nch w=1u l=180n
M2888 t1021 nw121 0 0 nch w=1u l=180n
M2889 t1019 nw231 vdd vdd pch w=2u l=180n
M2890 t1019 t1018 vdd vdd pch w=2u l=180n
CT1022 t1022 0 0.1f
M2891 t1019 nw231 t1022 0 nch w=1u l=180n
M2892 t1022 t1018 0 0 nch w=1u l=180n
M2893 t1020 nw121 vdd vdd pch w=2u l=180n
M2894 t1020 t1018 vdd vdd pch w=2u l=180n
CT1023 t1023 0 0.1f
M2895 t1020 nw121 t1023 0 nch w=1u l=180n
M2896 t1023 t1018 0 0 nch w=1u l=180n
M2897 nw426 t1019 vdd vdd pch w=2u l=180n
M2898 nw426 t1020 vdd vdd pch w=2u l=180n
CT1024 t1024 0 0.1f
M2899 nw426 t1019 t1024 0 nch w=1u l=180n
M2900 t1024 t1020 0 0 nch w=1u l=180n
Cnw426 nw426 0 2f
M2901 nw427 nw232 vdd vdd pch w=2u l=180n
M2902 nw427 nw122 vdd vdd pch w=2u l=180n
CT1025 t1025 0 0.1f
M2903 nw427 nw232 t1025 0 nch w=1u l=180n
M2904 t1025 nw122 0 0 nch w=1u l=180n
Cnw427 nw427 0 2f
M2905 nw428 nw233 0 0 nch w=1u l=180n
M2906 nw428 nw123 0 0 nch w=1u l=180n
CT1026 t1026 0 0.1f
M2907 t1026 nw233 vdd vdd pch w=2u l=180n
M2908 nw428 nw123 t1026 vdd pch w=2u l=180n
Cnw428 nw428 0 2f
CT1027 t1027 0 0.1f
M2909 t1027 nw234 vdd vdd pch w=2u l=180n
M2910 t1027 nw124 vdd vdd pch w=2u l=180n
CT1028 t1028 0 0.1f
M2911 t1027 nw234 t1028 0 nch w=1u l=180n
M2912 t1028 nw124 0 0 nch w=1u l=180n
M2913 nw429 t1027 vdd vdd pch w=2u l=180n
M2914 nw429 t1027 0 0 nch w=1u l=180n
Cnw429 nw429 0 2f
CT1029 t1029 0 0.1f
M2915 t1029 nw235 0 0 nch w=1u l=180n
M2916 t1029 nw125 0 0 nch w=1u l=180n
CT1030 t1030 0 0.1f
M2917 t1030 nw235 vdd vdd pch w=2u l=180n
M2918 t1029 nw125 t1030 vdd pch w=2u l=180n
M2919 nw430 t1029 vdd vdd pch w=2u l=180n
M2920 nw430 t1029 0 0 nch w=1u l=180n
Cnw430 nw430 0 2f
CT1031 t1031 0 0.1f
CT1032 t1032 0 0.1f
CT1033 t1033 0 0.1f
M2921 t1031 nw236 vdd vdd pch w=2u l=180n
M2922 t1031 nw126 vdd vdd pch w=2u l=180n
CT1034 t1034 0 0.1f
M2923 t1031 nw236 t1034 0 nch w=1u l=180n
M2924 t1034 nw126 0 0 nch w=1u l=180n
M2925 t1032 nw236 vdd vdd pch w=2u l=180n
M2926 t1032 t1031 vdd vdd pch w=2u l=180n
CT1035 t1035 0 0.1f
M2927 t1032 nw236 t1035 0 nch w=1u l=180n
M2928 t1035 t1031 0 0 nch w=1u l=180n
M2929 t1033 nw126 vdd vdd pch w=2u l=180n
M2930 t1033 t1031 vdd vdd pch w=2u l=180n
CT1036 t1036 0 0.1f
M2931 t1033 nw126 t1036 0 nch w=1u l=180n
M2932 t1036 t1031 0 0 nch w=1u l=180n
M2933 nw431 t1032 vdd vdd pch w=2u l=180n
M2934 nw431 t1033 vdd vdd pch w=2u l=180n
CT1037 t1037 0 0.1f
M2935 nw431 t1032 t1037 0 nch w=1u l=180n
M2936 t1037 t1033 0 0 nch w=1u l=180n
Cnw431 nw431 0 2f
M2937 nw432 nw237 vdd vdd pch w=2u l=180n
M2938 nw432 nw127 vdd vdd pch w=2u l=180n
CT1038 t1038 0 0.1f
M2939 nw432 nw237 t1038 0 nch w=1u l=180n
M2940 t1038 nw127 0 0 nch w=1u l=180n
Cnw432 nw432 0 2f
M2941 nw433 nw238 0 0 nch w=1u l=180n
M2942 nw433 nw128 0 0 nch w=1u l=180n
CT1039 t1039 0 0.1f
M2943 t1039 nw238 vdd vdd pch w=2u l=180n
M2944 nw433 nw128 t1039 vdd pch w=2u l=180n
Cnw433 nw433 0 2f
CT1040 t1040 0 0.1f
M2945 t1040 nw239 vdd vdd pch w=2u l=180n
M2946 t1040 nw129 vdd vdd pch w=2u l=180n
CT1041 t1041 0 0.1f
M2947 t1040 nw239 t1041 0 nch w=1u l=180n
M2948 t1041 nw129 0 0 nch w=1u l=180n
M2949 nw434 t1040 vdd vdd pch w=2u l=180n
M2950 nw434 t1040 0 0 nch w=1u l=180n
Cnw434 nw434 0 2f
CT1042 t1042 0 0.1f
M2951 t1042 nw240 0 0 nch w=1u l=180n
M2952 t1042 nw130 0 0 nch w=1u l=180n
CT1043 t1043 0 0.1f
M2953 t1043 nw240 vdd vdd pch w=2u l=180n
M2954 t1042 nw130 t1043 vdd pch w=2u l=180n
M2955 nw435 t1042 vdd vdd pch w=2u l=180n
M2956 nw435 t1042 0 0 nch w=1u l=180n
Cnw435 nw435 0 2f
CT1044 t1044 0 0.1f
CT1045 t1045 0 0.1f
CT1046 t1046 0 0.1f
M2957 t1044 nw241 vdd vdd pch w=2u l=180n
M2958 t1044 nw131 vdd vdd pch w=2u l=180n
CT1047 t1047 0 0.1f
M2959 t1044 nw241 t1047 0 nch w=1u l=180n
M2960 t1047 nw131 0 0 nch w=1u l=180n
M2961 t1045 nw241 vdd vdd pch w=2u l=180n
M2962 t1045 t1044 vdd vdd pch w=2u l=180n
CT1048 t1048 0 0.1f
M2963 t1045 nw241 t1048 0 nch w=1u l=180n
M2964 t1048 t1044 0 0 nch w=1u l=180n
M2965 t1046 nw131 vdd vdd pch w=2u l=180n
M2966 t1046 t1044 vdd vdd pch w=2u l=180n
CT1049 t1049 0 0.1f
M2967 t1046 nw131 t1049 0 nch w=1u l=180n
M2968 t1049 t1044 0 0 nch w=1u l=180n
M2969 nw436 t1045 vdd vdd pch w=2u l=180n
M2970 nw436 t1046 vdd vdd pch w=2u l=180n
CT1050 t1050 0 0.1f
M2971 nw436 t1045 t1050 0 nch w=1u l=180n
M2972 t1050 t1046 0 0 nch w=1u l=180n
Cnw436 nw436 0 2f
M2973 nw437 nw242 vdd vdd pch w=2u l=180n
M2974 nw437 nw132 vdd vdd pch w=2u l=180n
CT1051 t1051 0 0.1f
M2975 nw437 nw242 t1051 0 nch w=1u l=180n
M2976 t1051 nw132 0 0 nch w=1u l=180n
Cnw437 nw437 0 2f
M2977 nw438 nw243 0 0 nch w=1u l=180n
M2978 nw438 nw133 0 0 nch w=1u l=180n
CT1052 t1052 0 0.1f
M2979 t1052 nw243 vdd vdd pch w=2u l=180n
M2980 nw438 nw133 t1052 vdd pch w=2u l=180n
Cnw438 nw438 0 2f
CT1053 t1053 0 0.1f
M2981 t1053 nw244 vdd vdd pch w=2u l=180n
M2982 t1053 nw134 vdd vdd pch w=2u l=180n
CT1054 t1054 0 0.1f
M2983 t1053 nw244 t1054 0 nch w=1u l=180n
M2984 t1054 nw134 0 0 nch w=1u l=180n
M2985 nw439 t1053 vdd vdd pch w=2u l=180n
M2986 nw439 t1053 0 0 nch w=1u l=180n
Cnw439 nw439 0 2f
CT1055 t1055 0 0.1f
M2987 t1055 nw245 0 0 nch w=1u l=180n
M2988 t1055 nw135 0 0 nch w=1u l=180n
CT1056 t1056 0 0.1f
M2989 t1056 nw245 vdd vdd pch w=2u l=180n
M2990 t1055 nw135 t1056 vdd pch w=2u l=180n
M2991 nw440 t1055 vdd vdd pch w=2u l=180n
M2992 nw440 t1055 0 0 nch w=1u l=180n
Cnw440 nw440 0 2f
CT1057 t1057 0 0.1f
CT1058 t1058 0 0.1f
CT1059 t1059 0 0.1f
M2993 t1057 nw246 vdd vdd pch w=2u l=180n
M2994 t1057 nw136 vdd vdd pch w=2u l=180n
CT1060 t1060 0 0.1f
M2995 t1057 nw246 t1060 0 nch w=1u l=180n
M2996 t1060 nw136 0 0 nch w=1u l=180n
M2997 t1058 nw246 vdd vdd pch w=2u l=180n
M2998 t1058 t1057 vdd vdd pch w=2u l=180n
CT1061 t1061 0 0.1f
M2999 t1058 nw246 t1061 0 nch w=1u l=180n
M3000 t1061 t1057 0 0 nch w=1u l=180n
M3001 t1059 nw136 vdd vdd pch w=2u l=180n
M3002 t1059 t1057 vdd vdd pch w=2u l=180n
CT1062 t1062 0 0.1f
M3003 t1059 nw136 t1062 0 nch w=1u l=180n
M3004 t1062 t1057 0 0 nch w=1u l=180n
M3005 nw441 t1058 vdd vdd pch w=2u l=180n
M3006 nw441 t1059 vdd vdd pch w=2u l=180n
CT1063 t1063 0 0.1f
M3007 nw441 t1058 t1063 0 nch w=1u l=180n
M3008 t1063 t1059 0 0 nch w=1u l=180n
Cnw441 nw441 0 2f
M3009 nw442 nw247 vdd vdd pch w=2u l=180n
M3010 nw442 nw137 vdd vdd pch w=2u l=180n
CT1064 t1064 0 0.1f
M3011 nw442 nw247 t1064 0 nch w=1u l=180n
M3012 t1064 nw137 0 0 nch w=1u l=180n
Cnw442 nw442 0 2f
M3013 nw443 nw248 0 0 nch w=1u l=180n
M3014 nw443 nw138 0 0 nch w=1u l=180n
CT1065 t1065 0 0.1f
M3015 t1065 nw248 vdd vdd pch w=2u l=180n
M3016 nw443 nw138 t1065 vdd pch w=2u l=180n
Cnw443 nw443 0 2f
CT1066 t1066 0 0.1f
M3017 t1066 nw249 vdd vdd pch w=2u l=180n
M3018 t1066 nw139 vdd vdd pch w=2u l=180n
CT1067 t1067 0 0.1f
M3019 t1066 nw249 t1067 0 nch w=1u l=180n
M3020 t1067 nw139 0 0 nch w=1u l=180n
M3021 nw444 t1066 vdd vdd pch w=2u l=180n
M3022 nw444 t1066 0 0 nch w=1u l=180n
Cnw444 nw444 0 2f
CT1068 t1068 0 0.1f
M3023 t1068 nw250 0 0 nch w=1u l=180n
M3024 t1068 nw140 0 0 nch w=1u l=180n
CT1069 t1069 0 0.1f
M3025 t1069 nw250 vdd vdd pch w=2u l=180n
M3026 t1068 nw140 t1069 vdd pch w=2u l=180n
M3027 nw445 t1068 vdd vdd pch w=2u l=180n
M3028 nw445 t1068 0 0 nch w=1u l=180n
Cnw445 nw445 0 2f
CT1070 t1070 0 0.1f
CT1071 t1071 0 0.1f
CT1072 t1072 0 0.1f
M3029 t1070 nw251 vdd vdd pch w=2u l=180n
M3030 t1070 nw141 vdd vdd pch w=2u l=180n
CT1073 t1073 0 0.1f
M3031 t1070 nw251 t1073 0 nch w=1u l=180n
M3032 t1073 nw141 0 0 nch w=1u l=180n
M3033 t1071 nw251 vdd vdd pch w=2u l=180n
M3034 t1071 t1070 vdd vdd pch w=2u l=180n
CT1074 t1074 0 0.1f
M3035 t1071 nw251 t1074 0 nch w=1u l=180n
M3036 t1074 t1070 0 0 nch w=1u l=180n
M3037 t1072 nw141 vdd vdd pch w=2u l=180n
M3038 t1072 t1070 vdd vdd pch w=2u l=180n
CT1075 t1075 0 0.1f
M3039 t1072 nw141 t1075 0 nch w=1u l=180n
M3040 t1075 t1070 0 0 nch w=1u l=180n
M3041 nw446 t1071 vdd vdd pch w=2u l=180n
M3042 nw446 t1072 vdd vdd pch w=2u l=180n
CT1076 t1076 0 0.1f
M3043 nw446 t1071 t1076 0 nch w=1u l=180n
M3044 t1076 t1072 0 0 nch w=1u l=180n
Cnw446 nw446 0 2f
M3045 nw447 nw252 vdd vdd pch w=2u l=180n
M3046 nw447 nw142 vdd vdd pch w=2u l=180n
CT1077 t1077 0 0.1f
M3047 nw447 nw252 t1077 0 nch w=1u l=180n
M3048 t1077 nw142 0 0 nch w=1u l=180n
Cnw447 nw447 0 2f
M3049 nw448 nw253 0 0 nch w=1u l=180n
M3050 nw448 nw143 0 0 nch w=1u l=180n
CT1078 t1078 0 0.1f
M3051 t1078 nw253 vdd vdd pch w=2u l=180n
M3052 nw448 nw143 t1078 vdd pch w=2u l=180n
Cnw448 nw448 0 2f
CT1079 t1079 0 0.1f
M3053 t1079 nw254 vdd vdd pch w=2u l=180n
M3054 t1079 nw144 vdd vdd pch w=2u l=180n
CT1080 t1080 0 0.1f
M3055 t1079 nw254 t1080 0 nch w=1u l=180n
M3056 t1080 nw144 0 0 nch w=1u l=180n
M3057 nw449 t1079 vdd vdd pch w=2u l=180n
M3058 nw449 t1079 0 0 nch w=1u l=180n
Cnw449 nw449 0 2f
CT1081 t1081 0 0.1f
M3059 t1081 nw255 0 0 nch w=1u l=180n
M3060 t1081 nw145 0 0 nch w=1u l=180n
CT1082 t1082 0 0.1f
M3061 t1082 nw255 vdd vdd pch w=2u l=180n
M3062 t1081 nw145 t1082 vdd pch w=2u l=180n
M3063 nw450 t1081 vdd vdd pch w=2u l=180n
M3064 nw450 t1081 0 0 nch w=1u l=180n
Cnw450 nw450 0 2f
CT1083 t1083 0 0.1f
CT1084 t1084 0 0.1f
CT1085 t1085 0 0.1f
M3065 t1083 nw256 vdd vdd pch w=2u l=180n
M3066 t1083 nw146 vdd vdd pch w=2u l=180n
CT1086 t1086 0 0.1f
M3067 t1083 nw256 t1086 0 nch w=1u l=180n
M3068 t1086 nw146 0 0 nch w=1u l=180n
M3069 t1084 nw256 vdd vdd pch w=2u l=180n
M3070 t1084 t1083 vdd vdd pch w=2u l=180n
CT1087 t1087 0 0.1f
M3071 t1084 nw256 t1087 0 nch w=1u l=180n
M3072 t1087 t1083 0 0 nch w=1u l=180n
M3073 t1085 nw146 vdd vdd pch w=2u l=180n
M3074 t1085 t1083 vdd vdd pch w=2u l=180n
CT1088 t1088 0 0.1f
M3075 t1085 nw146 t1088 0 nch w=1u l=180n
M3076 t1088 t1083 0 0 nch w=1u l=180n
M3077 nw451 t1084 vdd vdd pch w=2u l=180n
M3078 nw451 t1085 vdd vdd pch w=2u l=180n
CT1089 t1089 0 0.1f
M3079 nw451 t1084 t1089 0 nch w=1u l=180n
M3080 t1089 t1085 0 0 nch w=1u l=180n
Cnw451 nw451 0 2f
M3081 nw452 nw257 vdd vdd pch w=2u l=180n
M3082 nw452 nw147 vdd vdd pch w=2u l=180n
CT1090 t1090 0 0.1f
M3083 nw452 nw257 t1090 0 nch w=1u l=180n
M3084 t1090 nw147 0 0 nch w=1u l=180n
Cnw452 nw452 0 2f
M3085 nw453 nw258 0 0 nch w=1u l=180n
M3086 nw453 nw148 0 0 nch w=1u l=180n
CT1091 t1091 0 0.1f
M3087 t1091 nw258 vdd vdd pch w=2u l=180n
M3088 nw453 nw148 t1091 vdd pch w=2u l=180n
Cnw453 nw453 0 2f
CT1092 t1092 0 0.1f
M3089 t1092 nw259 vdd vdd pch w=2u l=180n
M3090 t1092 nw149 vdd vdd pch w=2u l=180n
CT1093 t1093 0 0.1f
M3091 t1092 nw259 t1093 0 nch w=1u l=180n
M3092 t1093 nw149 0 0 nch w=1u l=180n
M3093 nw454 t1092 vdd vdd pch w=2u l=180n
M3094 nw454 t1092 0 0 nch w=1u l=180n
Cnw454 nw454 0 2f
CT1094 t1094 0 0.1f
M3095 t1094 nw260 0 0 nch w=1u l=180n
M3096 t1094 nw150 0 0 nch w=1u l=180n
CT1095 t1095 0 0.1f
M3097 t1095 nw260 vdd vdd pch w=2u l=180n
M3098 t1094 nw150 t1095 vdd pch w=2u l=180n
M3099 nw455 t1094 vdd vdd pch w=2u l=180n
M3100 nw455 t1094 0 0 nch w=1u l=180n
Cnw455 nw455 0 2f
CT1096 t1096 0 0.1f
CT1097 t1097 0 0.1f
CT1098 t1098 0 0.1f
M3101 t1096 nw261 vdd vdd pch w=2u l=180n
M3102 t1096 nw151 vdd vdd pch w=2u l=180n
CT1099 t1099 0 0.1f
M3103 t1096 nw261 t1099 0 nch w=1u l=180n
M3104 t1099 nw151 0 0 nch w=1u l=180n
M3105 t1097 nw261 vdd vdd pch w=2u l=180n
M3106 t1097 t1096 vdd vdd pch w=2u l=180n
CT1100 t1100 0 0.1f
M3107 t1097 nw261 t1100 0 nch w=1u l=180n
M3108 t1100 t1096 0 0 nch w=1u l=180n
M3109 t1098 nw151 vdd vdd pch w=2u l=180n
M3110 t1098 t1096 vdd vdd pch w=2u l=180n
CT1101 t1101 0 0.1f
M3111 t1098 nw151 t1101 0 nch w=1u l=180n
M3112 t1101 t1096 0 0 nch w=1u l=180n
M3113 nw456 t1097 vdd vdd pch w=2u l=180n
M3114 nw456 t1098 vdd vdd pch w=2u l=180n
CT1102 t1102 0 0.1f
M3115 nw456 t1097 t1102 0 nch w=1u l=180n
M3116 t1102 t1098 0 0 nch w=1u l=180n
Cnw456 nw456 0 2f
CT1103 t1103 0 0.1f
M3117 t1103 nw456 vdd vdd pch w=2u l=180n
M3118 t1103 nw456 0 0 nch w=1u l=180n
M3119 no0 t1103 vdd vdd pch w=2u l=180n
M3120 no0 t1103 0 0 nch w=1u l=180n
Cno0 no0 0 2f
CT1104 t1104 0 0.1f
M3121 t1104 nw455 vdd vdd pch w=2u l=180n
M3122 t1104 nw455 0 0 nch w=1u l=180n
M3123 no1 t1104 vdd vdd pch w=2u l=180n
M3124 no1 t1104 0 0 nch w=1u l=180n
Cno1 no1 0 2f
CT1105 t1105 0 0.1f
M3125 t1105 nw454 vdd vdd pch w=2u l=180n
M3126 t1105 nw454 0 0 nch w=1u l=180n
M3127 no2 t1105 vdd vdd pch w=2u l=180n
M3128 no2 t1105 0 0 nch w=1u l=180n
Cno2 no2 0 2f
CT1106 t1106 0 0.1f
M3129 t1106 nw453 vdd vdd pch w=2u l=180n
M3130 t1106 nw453 0 0 nch w=1u l=180n
M3131 no3 t1106 vdd vdd pch w=2u l=180n
M3132 no3 t1106 0 0 nch w=1u l=180n
Cno3 no3 0 2f
CT1107 t1107 0 0.1f
M3133 t1107 nw452 vdd vdd pch w=2u l=180n
M3134 t1107 nw452 0 0 nch w=1u l=180n
M3135 no4 t1107 vdd vdd pch w=2u l=180n
M3136 no4 t1107 0 0 nch w=1u l=180n
Cno4 no4 0 2f
CT1108 t1108 0 0.1f
M3137 t1108 nw451 vdd vdd pch w=2u l=180n
M3138 t1108 nw451 0 0 nch w=1u l=180n
M3139 no5 t1108 vdd vdd pch w=2u l=180n
M3140 no5 t1108 0 0 nch w=1u l=180n
Cno5 no5 0 2f
CT1109 t1109 0 0.1f
M3141 t1109 nw450 vdd vdd pch w=2u l=180n
M3142 t1109 nw450 0 0 nch w=1u l=180n
M3143 no6 t1109 vdd vdd pch w=2u l=180n
M3144 no6 t1109 0 0 nch w=1u l=180n
Cno6 no6 0 2f
CT1110 t1110 0 0.1f
M3145 t1110 nw449 vdd vdd pch w=2u l=180n
M3146 t1110 nw449 0 0 nch w=1u l=180n
M3147 no7 t1110 vdd vdd pch w=2u l=180n
M3148 no7 t1110 0 0 nch w=1u l=180n
Cno7 no7 0 2f
.model nch NMOS (vto=0.45 kp=200u lambda=0.05)
.model pch PMOS (vto=-0.45 kp=100u lambda=0.05)
* outputs: nw4 nw8 nw12 nw16 nw20 nw24 nw28 nw32 nw36 nw40 nw44 nw48 nw52 nw56 nw60 nw64 nw68 nw72 nw76 no0 no1 no2 no3 no4 no5 no6 no7
.end
